/*
 * sparsedrop.h — C ABI of libsparsedrop.so, the sm_100a SparseDrop engine.
 *
 * Every entry point is plain C: raw device pointers, sizes, element strides and a
 * CUDA stream handle passed as void*.  No torch types, no exceptions.  All functions
 * that launch work are asynchronous on the given stream, allocate nothing on the
 * device, and return SD_OK (0) or a negative sd_status code; sd_last_error() gives the
 * message of the most recent failure on the calling thread.
 *
 * Each declaration cites the interface of andylolu2/sparse-dropout that it replaces
 * (paths are relative to that project's root).
 *
 * Matrix convention (same as the reference extension):  A is [M, K], B is [N, K],
 * C = scale * (A . B^T) is [M, N].  A matrix is described by its pointer plus the element
 * strides of its two logical dimensions (row stride, column stride); exactly one of the
 * two strides must be 1 ("row-major" when the column stride is 1, "column-major" when the
 * row stride is 1), which is the operand rule of flash_dropout/cuda/src/gemm_binding.cu:18-22.
 * The non-unit stride must be a multiple of 8 elements and the pointer 16-byte aligned
 * (TMA requirement).  M, N, K need not be multiples of the block size: blocks at the ragged
 * edge are zero-padded logically (the reference asserts divisibility instead,
 * flash_dropout/cuda/src/matmul_dsd.cuh:87-95).
 */
#ifndef SPARSEDROP_H_
#define SPARSEDROP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sd_status {
    SD_OK = 0,
    SD_ERR_INVALID_ARG = -1,   /* null pointer, bad size, p outside [0,1), bad dtype ... */
    SD_ERR_LAYOUT = -2,        /* neither stride is 1, or stride / pointer not TMA-aligned */
    SD_ERR_CUDA = -3,          /* a CUDA runtime / driver call failed */
    SD_ERR_TIMEOUT = -4,       /* a device-side bounded wait expired (read by sd_check_status) */
    SD_ERR_TOO_LARGE = -5      /* size beyond a documented maximum */
} sd_status;

typedef enum sd_dtype {
    SD_F16 = 0,                /* IEEE half   (the only dtype of gemm_binding.cu:49-50) */
    SD_BF16 = 1,               /* bfloat16    (extension: the reference is fp16-only)   */
    SD_F32 = 2                 /* float: only as the output / gradient dtype of sd_layernorm_* */
} sd_dtype;

/* Side of the block plan a DSD product reduces over. */
typedef enum sd_plan_side {
    SD_PLAN_ROWS = 0,          /* A's row-blocks are the plan's rows  (forward,  mask)   */
    SD_PLAN_COLS = 1           /* A's row-blocks are the plan's columns (dW, i.e. mask.T) */
} sd_plan_side;

/* Library version (major*10000 + minor*100 + patch). */
int sd_version(void);

/* Message of the last error raised on this thread ("" if none). */
const char* sd_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Block plan = the drop mask plus every compacted kept-block index list the kernels walk.
 *
 * A plan describes an R x C grid of 128x128 tiles (R = ceil(M/128), C = ceil(K/128)).  The
 * logical dropout blocks may be larger, and need not be square: block_size = (128*rep_r, 128*rep_c) — the (m, k)
 * pairs of eval/mlp/config.py:23-27 — and tile (r, c) inherits the decision of logical block
 * (r / rep_r, c / rep_c).  True / 1 = dropped, as in
 * flash_dropout/functional/utils.py:11-16.
 *
 * The plan lives in ONE caller-allocated device buffer of sd_plan_bytes(R, C) bytes, laid out
 * as int32 arrays at the offsets reported by sd_plan_offsets():
 *   header[16]   : [0] nnz kept tiles, [1] number of SDD work items, [2] number of dropped
 *                  tiles, [3] R, [4] C, [5] max kept per row, [6] max kept per column
 *   row_ptr[R+1], col_idx[R*C]   : CSR of kept tiles (kept column indices per row, ascending)
 *   col_ptr[C+1], row_idx[R*C]   : CSC of kept tiles (kept row indices per column, ascending)
 *   kept_pairs[2*R*C]            : (row, col) of kept tiles in row-major order — the order of
 *                                  torch.nonzero(~mask) used by
 *                                  flash_dropout/functional/blockwise_dropout_matmul_triton.py:48
 *   drop_pairs[2*R*C]            : (row, col) of dropped tiles in row-major order
 *   row_order[R], col_order[C]   : permutations, most kept tiles first
 *   sdd_items[3*R*ceil(C/2)]     : (row, col0, col1 or -1): kept tiles of one row paired up
 *   mask[R*C] (uint8)            : 1 = dropped, row-major, tile granularity
 * ------------------------------------------------------------------------------------------ */
typedef struct sd_plan_layout {
    int64_t header, row_ptr, col_idx, col_ptr, row_idx, kept_pairs, drop_pairs,
            row_order, col_order, sdd_items, mask, total_bytes;   /* byte offsets */
} sd_plan_layout;

size_t sd_plan_bytes(int R, int C);
int sd_plan_offsets(int R, int C, sd_plan_layout* out);

/*
 * Draw the Bernoulli(p) drop mask on the device and build the plan in one launch.
 * Replaces blockwise_dropout_mask (flash_dropout/functional/utils.py:11-16: torch.rand(...) < p)
 * and the index-list builders (utils.py:19-69 mask_to_increment_table;
 * blockwise_dropout_matmul_triton.py:48 torch.nonzero(~mask)).
 * Logical block (i, j) of the ceil(R/rep_r) x ceil(C/rep_c) grid (Cm = ceil(C/rep_c) columns) is dropped iff
 *   u < p,  u = float(philox4x32_10(key = seed, counter = (i*Cm + j, 0, offset_lo, offset_hi)).x >> 8) * 2^-24
 * compared in fp32.  mask_out (optional, may be NULL) receives the logical mask as
 * ceil(R/rep_r) x ceil(C/rep_c) bytes, row-major.
 */
int sd_plan_from_seed(void* plan, int R, int C, int rep_r, int rep_c, uint64_t seed, uint64_t offset, float p,
                      uint8_t* mask_out, void* stream);

/*
 * Same draw, but the offset is base_offset + *device_counter, read on the device, and the launch
 * increments *device_counter (a uint64 in device memory).  The host no longer chooses the offset, so a
 * captured CUDA graph that contains this launch draws a fresh mask on every replay.  No counterpart in
 * the reference (its masks come from torch.rand on the host-controlled generator, utils.py:15).
 */
int sd_plan_from_seed_counter(void* plan, int R, int C, int rep_r, int rep_c, uint64_t seed, uint64_t base_offset,
                              uint64_t* device_counter, float p, uint8_t* mask_out, void* stream);

/*
 * Several plans from ONE launch: plan i of n draws like sd_plan_from_seed_counter with offset base_offset + i +
 * *device_counter, and the launch advances the shared counter by n, so the masks equal those of n single launches
 * in that order.  The descriptors live in a caller-owned device buffer of sd_plan_batch_desc_bytes(n) bytes, zero
 * initialised, 8-byte aligned: fill a host buffer of the same size entry by entry with sd_plan_batch_describe
 * (which needs the device buffer's address), copy it to the device once, then call sd_plan_batch_launch every step.
 * Each plan is at most 3072 x 32 tiles.  No counterpart in the reference (one torch.rand call per layer per step,
 * flash_dropout/functional/utils.py:15).
 */
size_t sd_plan_batch_desc_bytes(int n);
int sd_plan_batch_describe(void* host_desc, void* device_desc, int n, int i, void* plan, int R, int C, int rep_r, int rep_c,
                           uint64_t seed, uint64_t base_offset, uint64_t* device_counter, float p, uint8_t* mask_out);
int sd_plan_batch_launch(const void* device_desc, int n, void* stream);

/*
 * Build the plan from a caller-supplied bool mask (1 byte per logical block, any two strides),
 * the form in which the reference passes masks to gemm_dsd / gemm_sdd
 * (flash_dropout/cuda/binding_gemm.py:29-47).  mask is ceil(R/rep_r) x ceil(C/rep_c).
 */
int sd_plan_from_mask(void* plan, int R, int C, int rep_r, int rep_c, const uint8_t* mask,
                      int64_t mask_row_stride, int64_t mask_col_stride, void* stream);

/* ------------------------------------------------------------------------------------------
 * GEMMs.  `status` is an optional device int32 (may be NULL) that a kernel sets to a non-zero
 * code if one of its bounded waits expires; sd_check_status() copies it back and translates.
 *
 * `workspace` is optional device scratch (may be NULL).  A launch with fewer 128x256 output tiles
 * than SMs (small layers; the dW product of a conv, whose reduction runs over all N*P*Q rows) would
 * leave SMs idle if tiles were handed out whole, so with a workspace (and a reduction of at least
 * 16 K tiles) it gives every output tile a group of SMs instead, sized in proportion to the tile's
 * kept K tiles: each CTA of a group computes one part of the tile's reduction and parks its fp32
 * partial tile in the workspace, and the CTAs of the group each add up a different part of the
 * tile over all partials (in CTA order, so results are reproducible).  Launches with enough tiles
 * never touch the workspace.  It is
 * sd_workspace_bytes() bytes for the current device (8 KiB of counters + 128 KiB per SM, 18.5 MiB
 * on a B200), 16-byte aligned, and must be passed through
 * sd_workspace_init() once before its first use (and again after a launch that reported
 * SD_ERR_TIMEOUT).  A launch leaves the flags cleared.  Launches that may overlap on the GPU
 * (different streams) need different workspaces.  No counterpart in the reference, whose kernels
 * use a fixed one-CTA-per-tile grid (flash_dropout/cuda/src/matmul_dsd.cuh:99-105).
 * ------------------------------------------------------------------------------------------ */
size_t sd_workspace_bytes(void);
int sd_workspace_init(void* workspace, void* stream);

/* SMs that every GEMM / conv launch made after this call leaves free (default 0, or the value of the environment
 * variable SD_SM_MARGIN when the library is loaded); returns the previous value, or SD_ERR_INVALID_ARG for a
 * negative one.  The kernels are persistent, one CTA per SM for the whole launch with tiles dealt out up front:
 * when another kernel (a gradient all-reduce that overlaps the next step) occupies SMs, CTAs that have to wait for
 * one stretch the launch by up to a whole pass, while the other kernel crawls for lack of SMs.  A margin of about
 * as many SMs as that kernel has CTAs lets both run side by side; launches that do not fill the GPU anyway are
 * unaffected.  Process-wide; no counterpart in the reference (one CTA per tile, flash_dropout/cuda/src/matmul_dsd.cuh:99-105). */
int sd_set_sm_margin(int sms);

/* Dense C = scale * A . B^T.  Replaces GEMM.gemm (flash_dropout/cuda/binding_gemm.py:26-27,
 * flash_dropout/cuda/src/gemm.cuh:143-167). */
int sd_gemm(const void* A, int64_t a_rs, int64_t a_cs,
            const void* B, int64_t b_rs, int64_t b_cs,
            void* C, int64_t c_rs, int64_t c_cs,
            int M, int N, int K, float scale, int dtype, void* workspace, int* status, void* stream);

/* DSD: C = scale * (keep o A) . B^T, skipping dropped 128-wide K tiles of each 128-row block
 * of A.  Replaces GEMM.gemm_dsd (flash_dropout/cuda/binding_gemm.py:29-37,
 * flash_dropout/cuda/src/matmul_dsd.cuh:70-106).  With side = SD_PLAN_ROWS the plan is
 * R = ceil(M/128) x C = ceil(K/128) (forward); with SD_PLAN_COLS it is ceil(K/128) x ceil(M/128)
 * (A = x^T, the dW product of flash_dropout/functional/blockwise_dropout_matmul_cuda.py:47-51).
 * Row-blocks with no kept tile produce zeros. */
int sd_gemm_dsd(const void* A, int64_t a_rs, int64_t a_cs,
                const void* B, int64_t b_rs, int64_t b_cs,
                void* C, int64_t c_rs, int64_t c_cs,
                int M, int N, int K, const void* plan, int plan_side,
                float scale, int dtype, void* workspace, int* status, void* stream);

/*
 * DSD without a caller workspace and without any allocation.  No counterpart in the reference.
 *
 * For callers that cannot hand this library device memory of their own: a host process whose device
 * memory all belongs to its own pool or fixed budget, a latency-bound loop that must not take the
 * device-wide synchronisation an allocation implies, or a plain C caller with no allocator at hand.
 * sd_gemm_dsd() needs such a caller to allocate the workspace before it can spread a small product over
 * all SMs; this entry point computes the same product with scratch that is built into the library:
 * a file-scope device array of 8 200 KiB (8 KiB of counters + 64 partial tiles of 128 KiB) that every GPU
 * which loads the library holds until the process exits.  It calls no cudaMalloc / cudaFree and no
 * allocating library routine; inputs, the plan and the output are still the caller's.
 *
 * Limit: at most 64 output tiles of 128 x 256, i.e. ceil(M/128) * ceil(N/256) <= 64 (a 1024 x 2048
 * result, say); the grid is at most 64 CTAs.  Larger products return SD_ERR_TOO_LARGE — they have at
 * least one tile per CTA and need no scratch: use sd_gemm_dsd() with workspace = NULL.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and keeps it; make that first call outside any stream capture.  Every call on a
 * device shares the one array: its counters are cleared on the stream at the start of each call, and two
 * calls that can overlap on the GPU (different streams, different threads) race on it — serialise them.
 */
int sd_gemm_dsd_static_scratch(const void* A, int64_t a_rs, int64_t a_cs,
                               const void* B, int64_t b_rs, int64_t b_cs,
                               void* C, int64_t c_rs, int64_t c_cs,
                               int M, int N, int K, const void* plan, int plan_side,
                               float scale, int dtype, int* status, void* stream);

/* SDD: C = scale * keep o (A . B^T): only kept 128x128 output tiles are computed, dropped tiles
 * are written as zeros.  The plan is ceil(M/128) x ceil(N/128).  Replaces GEMM.gemm_sdd
 * (flash_dropout/cuda/binding_gemm.py:39-47, flash_dropout/cuda/src/matmul_sdd.cuh:69-105). */
int sd_gemm_sdd(const void* A, int64_t a_rs, int64_t a_cs,
                const void* B, int64_t b_rs, int64_t b_cs,
                void* C, int64_t c_rs, int64_t c_cs,
                int M, int N, int K, const void* plan,
                float scale, int dtype, void* workspace, int* status, void* stream);

/* Same as sd_gemm_sdd but dropped tiles of C are left untouched instead of being zero-filled, for
 * consumers that read kept tiles only (sd_col2im_kept): saves writing the dropped share of C.
 * No counterpart in the reference. */
int sd_gemm_sdd_kept(const void* A, int64_t a_rs, int64_t a_cs,
                     const void* B, int64_t b_rs, int64_t b_cs,
                     void* C, int64_t c_rs, int64_t c_cs,
                     int M, int N, int K, const void* plan,
                     float scale, int dtype, void* workspace, int* status, void* stream);

/* Same as sd_gemm_sdd_kept for a plan that describes the TRANSPOSE of the result: the plan's grid is
 * ceil(N/128) x ceil(M/128) and its kept pair (r, c) is the result's 128x128 tile (c, r).  One tile per
 * work item.  The convolution's input gradient uses it to produce the K-outer matrix dcolT[K, M] =
 * W^T . dY^T row-major (a plain TMA store) from the plan of the M x K im2col matrix, instead of
 * computing dcol[M, K] and storing it transposed.  No counterpart in the reference. */
int sd_gemm_sdd_kept_t(const void* A, int64_t a_rs, int64_t a_cs,
                       const void* B, int64_t b_rs, int64_t b_cs,
                       void* C, int64_t c_rs, int64_t c_cs,
                       int M, int N, int K, const void* plan,
                       float scale, int dtype, void* workspace, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Convolution stages.  The im2col matrix of flash_dropout/functional/im2col_conv2d.py:17-20
 * (M = N*P*Q rows, K = C*R*S columns, k = c*R*S + r*S + s) is kept K-outer: colT[k][m], 16-bit,
 * leading dimension ldm (>= M, multiple of 8, base 16-byte aligned), with k_gemm >= K rows
 * (k_gemm = the K the GEMMs are called with, a multiple of 8; rows K..k_gemm-1 must be zero).
 * colT.T is the MN-major A operand of sd_gemm_dsd; the plan is ceil(M/128) x ceil(k_gemm/128).
 * x and dx are contiguous NCHW.  Blockwise dropout on a convolution has no counterpart in the
 * reference (flash_dropout/layers/dropout_conv.py:86-99 is commented out); the dense im2col it
 * replaces is F.unfold in im2col_conv2d.py:17.
 * ------------------------------------------------------------------------------------------ */

/* Writes the kept 128x128 blocks of colT (all blocks if plan is NULL).  Dropped blocks are not touched. */
int sd_im2col_kept(const void* x, int N, int C, int H, int W, int R, int S,
                   int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                   void* colT, int64_t ldm, int k_gemm, const void* plan, void* stream);

/* Adjoint: dx[n,c,h,w] = sum of the dcolT entries that x[n,c,h,w] fed, reading kept blocks only
 * (all blocks if plan is NULL).  fp32 accumulation, output in `dtype`. */
int sd_col2im_kept(const void* dcolT, int64_t ldm, int k_gemm, int N, int C, int H, int W, int R, int S,
                   int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                   void* dx, const void* plan, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Panel layout of the im2col matrix: [ceil(M/128)][k_gemm][128] — panel b holds pixels m = 128*b ..
 * 128*b+127, its row k their k-th im2col entries — so a kept 128x128 block is one contiguous 32 KB
 * run instead of 128 runs of 256 bytes at a stride of ldm.  k_gemm must be a multiple of 64 (rows
 * K..k_gemm-1 zero), the base 16-byte aligned; the plan is ceil(M/128) x ceil(k_gemm/128) as before.
 * The four functions below are the panel forms of sd_im2col_kept, sd_col2im_kept, sd_gemm_dsd with the
 * im2col matrix as its A operand, and sd_gemm_sdd_kept_t with it as the result.  No counterpart in the
 * reference.
 * ------------------------------------------------------------------------------------------ */
int sd_im2col_kept_panels(const void* x, int N, int C, int H, int W, int R, int S,
                          int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                          void* col_panels, int k_gemm, const void* plan, void* stream);

int sd_col2im_kept_panels(const void* dcol_panels, int k_gemm, int N, int C, int H, int W, int R, int S,
                          int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                          void* dx, const void* plan, int dtype, void* stream);

/* DSD with the panel matrix P (pixels x kg) as A.  SD_PLAN_ROWS: C[pixels, N] = scale * (keep o col) . B^T with
 * B[N, kg] (the convolution's forward); SD_PLAN_COLS: C[kg, N] = scale * (keep o col)^T . B^T with B[N, pixels]
 * (its weight gradient). */
int sd_gemm_dsd_panels(const void* P, int pixels, int kg,
                       const void* B, int64_t b_rs, int64_t b_cs,
                       void* C, int64_t c_rs, int64_t c_cs, int N,
                       const void* plan, int plan_side,
                       float scale, int dtype, void* workspace, int* status, void* stream);

/* Kept tiles of P[kg, pixels] = scale * A . B^T (A[kg, K], B[pixels, K]) written into the panel matrix P; the
 * plan is the one of the pixels x kg matrix (sd_gemm_sdd_kept_t).  Dropped blocks of P are left untouched. */
int sd_gemm_sdd_kept_t_panels(const void* A, int64_t a_rs, int64_t a_cs,
                              const void* B, int64_t b_rs, int64_t b_cs,
                              void* P, int kg, int pixels, int K, const void* plan,
                              float scale, int dtype, void* workspace, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Products with an elementwise neighbour of the layer fused into the epilogue.  The reference applies these as
 * separate PyTorch ops around DropoutMM: ReLU after every layer of its MLP (eval/mlp/model.py:33-38), and autograd's
 * cast + accumulate of the 16-bit weight gradient into the fp32 parameter gradient
 * (flash_dropout/functional/blockwise_dropout_matmul_cuda.py:35-53 under autocast).
 * ------------------------------------------------------------------------------------------ */

/* sd_gemm_dsd whose result goes through ReLU before it is stored: C = max(scale * (keep o A) . B^T, 0). */
int sd_gemm_dsd_relu(const void* A, int64_t a_rs, int64_t a_cs,
                     const void* B, int64_t b_rs, int64_t b_cs,
                     void* C, int64_t c_rs, int64_t c_cs,
                     int M, int N, int K, const void* plan, int plan_side,
                     float scale, int dtype, void* workspace, int* status, void* stream);

/* sd_gemm_dsd with an fp32 result: C (float, element strides c_rs / c_cs, 4-byte aligned) is overwritten, or with
 * accumulate != 0 added to.  For the weight gradient: written straight into the fp32 gradient of the parameter. */
int sd_gemm_dsd_f32(const void* A, int64_t a_rs, int64_t a_cs,
                    const void* B, int64_t b_rs, int64_t b_cs,
                    float* C, int64_t c_rs, int64_t c_cs,
                    int M, int N, int K, const void* plan, int plan_side,
                    float scale, int dtype, int accumulate, void* workspace, int* status, void* stream);

/* sd_gemm_sdd followed by the derivative of a ReLU that produced the layer's input X[M, N] (row-major, row stride
 * x_rs, 16-byte aligned rows, N a multiple of 8): C = (X > 0) o scale * keep o (A . B^T). */
int sd_gemm_sdd_relu_mask(const void* A, int64_t a_rs, int64_t a_cs,
                          const void* B, int64_t b_rs, int64_t b_cs,
                          void* C, int64_t c_rs, int64_t c_cs,
                          int M, int N, int K, const void* plan,
                          const void* X, int64_t x_rs,
                          float scale, int dtype, void* workspace, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused convolution: im2col + DSD in one kernel.  The A operand of the product is the im2col matrix of
 * flash_dropout/functional/im2col_conv2d.py:17-20 (rows = output pixels m = (n, p, q), columns k = c*R*S + r*S + s),
 * but it is never written to memory: extra warps of the GEMM kernel gather each 64-wide stage of it straight from
 * the contiguous NCHW input x into shared memory, and only the kept blocks of the plan are ever gathered.  The plan
 * is the one of the N*P*Q x C*R*S matrix, ceil(N*P*Q/128) x ceil(C*R*S/128).  Served geometries (ask
 * sd_conv_fused_supported; other geometries use the sd_im2col_kept path): S = 3, unit horizontal stride and
 * dilation, pad_w = 1, W in {8, 16, 32, 64}; any R, vertical stride, dilation and padding.  No counterpart in the
 * reference, whose conv layer materialises the matrix with F.unfold (im2col_conv2d.py:17) and has no blockwise
 * dropout (flash_dropout/layers/dropout_conv.py:86-99 is commented out).
 * ------------------------------------------------------------------------------------------ */

/* 1 if the geometry is served by sd_conv_dsd_fwd / sd_conv_dsd_dw, else 0. */
int sd_conv_fused_supported(int N, int C, int H, int W, int R, int S,
                            int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w);

/* Forward: Y2d[N*P*Q, Ko] = scale * (keep o im2col(x)) . W2d^T with W2d[Ko, >= C*R*S] (the filter viewed 2-D;
 * columns past C*R*S are never read).  Y2d viewed (N, P, Q, Ko) is the channels-last result. */
int sd_conv_dsd_fwd(const void* x, int N, int C, int H, int W, int R, int S,
                    int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                    const void* W2d, int64_t w_rs, int64_t w_cs,
                    void* Y2d, int64_t y_rs, int64_t y_cs, int Ko,
                    const void* plan, float scale, int dtype, void* workspace, int* status, void* stream);

/* Weight gradient: dW2d[Ko, C*R*S] = scale * dY2d^T . (keep o im2col(x)) with dY2d[N*P*Q, Ko]; columns of dW2d
 * past C*R*S (if its row stride leaves room for any) are not written.  Reduces over all pixels: pass a workspace. */
int sd_conv_dsd_dw(const void* x, int N, int C, int H, int W, int R, int S,
                   int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                   const void* dY2d, int64_t dy_rs, int64_t dy_cs,
                   void* dW2d, int64_t dw_rs, int64_t dw_cs, int Ko,
                   const void* plan, float scale, int dtype, void* workspace, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * LayerNorm over the last dimension of x[rows, n] (fp32, contiguous, n a multiple of 4 and at most 1024), for the
 * normalisations that sit in front of the SparseDrop layers of the transformer consumers.  The reference uses
 * torch.nn.LayerNorm there (eval/llm/model.py:72-74,113; eval/vit/model.py:11,53,106-108), whose result autocast then
 * casts to 16 bits for the DropoutMM that follows; no counterpart among the reference's own kernels.
 *   forward : y = (x - mean) * rstd * gamma (+ beta, may be NULL), rstd = 1 / sqrt(var + eps), biased variance;
 *             y is written as y_dtype (SD_F32, SD_BF16 or SD_F16); mean[rows] and rstd[rows] are kept for backward.
 *   backward: dx[rows, n] (fp32), and dgamma[n] / dbeta[n] (dbeta may be NULL) overwritten or, with accumulate != 0,
 *             added to; dy is read as dy_dtype.  workspace: sd_layernorm_bwd_workspace_bytes(rows, n) bytes,
 *             16-byte aligned (per-CTA partial sums of the two parameter gradients).
 * ------------------------------------------------------------------------------------------ */
int sd_layernorm_fwd(const float* x, int rows, int n, const float* gamma, const float* beta, float eps, void* y,
                     int y_dtype, float* mean, float* rstd, void* stream);
size_t sd_layernorm_bwd_workspace_bytes(int rows, int n);
int sd_layernorm_bwd(const float* x, const void* dy, int dy_dtype, const float* gamma, const float* mean,
                     const float* rstd, int rows, int n, float* dx, float* dgamma, float* dbeta, int accumulate,
                     void* workspace, void* stream);

/*
 * Exercises the bounded device-side waits the kernels are built on, without a fault or a hang: a one-warp kernel
 * waits on a barrier nobody arrives on and on a counter nobody increments, each for at most limit_ns (<= 1 s),
 * gives up, and returns normally.  `words` is 4 device ints: [0] status word (first give-up code, 101),
 * [1] the counter that stays 0, [2] bit mask (1|2 = a wait wrongly succeeded, 4|8 = its abort flag was raised),
 * [3] elapsed microseconds.  sd_check_status(words, stream) then reports SD_ERR_TIMEOUT.  No counterpart in the
 * reference, whose kernels have no waits to bound.
 */
int sd_selftest_bounded_wait(int* words, uint64_t limit_ns, void* stream);

/* Synchronises the stream, reads *status and returns SD_OK or SD_ERR_TIMEOUT. */
int sd_check_status(const int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSEDROP_H_ */
