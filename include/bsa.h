/* bsa.h -- C ABI of the B200 block-sparse attention library (libbsa_b200.so).
 *
 * The reference (linxihui/dkernel) has no FFI: its device boundary is a set of
 * Triton launches made from Python.  Each entry point below replaces one of
 * those launch sites (cited per function, paths relative to the reference
 * project).  The host package calls them through ctypes.
 *
 * Conventions
 *  - Every pointer is a device pointer owned by the caller (PyTorch allocates
 *    inputs, outputs, layouts and workspaces); the library never allocates or
 *    frees device memory and never synchronises.  Work is enqueued on `stream`
 *    (a cudaStream_t passed as void*).
 *  - Strides are in ELEMENTS, the head dimension is contiguous (stride 1).
 *  - Return value: 0 on success, a negative BSA_E_* code otherwise; the text of
 *    the last error of the calling thread is available from bsa_last_error().
 *    Nothing aborts, traps or throws across the boundary.
 *  - Thread safety: entry points may be called concurrently from several host
 *    threads and for several devices; the current CUDA device of the calling
 *    thread must be the one that owns the pointers.
 */
#ifndef BSA_B200_H_
#define BSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSA_ABI_VERSION 3

enum {
  BSA_OK = 0,
  BSA_E_BADARG = -1,      /* null pointer, negative size, inconsistent shapes   */
  BSA_E_UNSUPPORTED = -2, /* shape / dtype / stride not handled by any kernel   */
  BSA_E_CUDA = -3,        /* a CUDA runtime or driver call failed               */
  BSA_E_TOOBIG = -4       /* problem exceeds a documented fixed limit           */
};

enum { BSA_F16 = 0, BSA_BF16 = 1, BSA_F32 = 2, BSA_F8E4M3 = 3 /* K/V storage of bsa_decode only */ };

/* which kernel family serves a call */
enum { BSA_IMPL_AUTO = 0, BSA_IMPL_GENERIC = 1, BSA_IMPL_SM100 = 2 };

/* how the pattern row of a query tile is chosen */
enum {
  BSA_ROWS_BY_TILE = 0,    /* row = q tile index (training path,
                              dkernel/ops/sparse_attn_fwd.py:289-291)           */
  BSA_ROWS_BY_POSITION = 1 /* row = (past_len + tile start) / block, positions
                              re-based per sequence (inference path,
                              dkernel/ops/sparse_attn_inference.py:503-514)     */
};

int bsa_abi_version(void);
const char* bsa_last_error(void);

/* ---------------------------------------------------------------------------
 * Sparse-layout builder.  Replaces the CPU/numpy round trip of
 * dkernel/utils.py:105-229 (get_sparse_attn_mask) and :19-65,:91-95
 * (dense_to_crow_col / dense_to_ccol_row).
 * ------------------------------------------------------------------------- */
typedef struct {
  int32_t num_heads;          /* q heads described (rows of the mask's head axis) */
  int32_t num_kv_heads;       /* <= num_heads, divides it                         */
  int32_t num_dense_heads;    /* last kv heads that are dense                     */
  int32_t q_blocks;           /* rows of the block mask before trimming           */
  int32_t kv_blocks;
  int32_t q_start_block;      /* q_start_position / block_size                    */
  int32_t kv_start_block;     /* kv_start_position / block_size                   */
  int32_t trim_q_blocks;      /* cdiv(past_len, block_size): rows dropped on top  */
  int32_t local_left;         /* local_blocks (left, including the diagonal)      */
  int32_t local_right;        /* 1 when causal                                    */
  int32_t vert_stride;
  int32_t head_sliding_step;  /* already resolved: max(1, vert_stride/num_heads)  */
  int32_t head_sliding_offset;
  int32_t causal;
  int32_t absolute_vert;      /* 1 = absolute vertical positions, 0 = relative    */
} bsa_local_stride_params;

/* Writes the uint8 block mask (num_heads, q_blocks - trim_q_blocks, kv_blocks),
 * contiguous.  dkernel/utils.py:182-220. */
int bsa_local_stride_mask(const bsa_local_stride_params* p, uint8_t* mask, void* stream);

/* CSR row pointers of a (H, M, N) uint8 mask with arbitrary element strides:
 * crow (H, M+1) int32 contiguous, nnz (H,) int32 = crow[:, M].
 * For the CSC layout pass the mask with its last two strides swapped.
 * dkernel/utils.py:19-24 (to_csr: cumsum of row counts). */
int bsa_csr_row_ptr(const uint8_t* mask, int32_t H, int32_t M, int32_t N,
                    int64_t stride_h, int64_t stride_m, int64_t stride_n,
                    int32_t* crow, int32_t* nnz, void* stream);

/* Column indices in row-major order, every head padded with -1 up to `width`
 * entries (width >= max nnz).  With val != NULL the value of each non-zero is
 * stored too (0 in the padding): the (col, value) pairs of
 * dense_to_crow_col(include_values=True) are written interleaved when
 * interleave_values != 0 (col has 2*width ints per head).
 * dkernel/utils.py:47-61. */
int bsa_csr_fill_cols(const uint8_t* mask, int32_t H, int32_t M, int32_t N,
                      int64_t stride_h, int64_t stride_m, int64_t stride_n,
                      const int32_t* crow, int32_t* col, int32_t width,
                      int32_t interleave_values, void* stream);

/* ---------------------------------------------------------------------------
 * Attention forward.  Replaces the launches of _sparse_fwd_kernel
 * (dkernel/ops/sparse_attn_fwd.py:519-546) and _fwd_kernel_batch_inference
 * (dkernel/ops/sparse_attn_inference.py:113-145, :245-285).
 * ------------------------------------------------------------------------- */
typedef struct {
  const void* q; const void* k; const void* v; void* o;
  float* lse;                 /* may be NULL; natural-log LSE of scaled logits  */
  int64_t q_sb, q_ss, q_sh;   /* batch / sequence / head strides                */
  int64_t k_sb, k_ss, k_sh;
  int64_t v_sb, v_ss, v_sh;
  int64_t o_sb, o_ss, o_sh;
  int64_t lse_sb, lse_sh;     /* LSE sequence stride is 1                       */
  int32_t batch, hq, hkv, d;
  int32_t sq, sk;             /* storage lengths of the sequence axis           */
  int32_t total_q;            /* packed batch: upper bound of sum(q lengths); the
                                 q tiles of all sequences are then enumerated
                                 back to back.  0 = dense (batch, sq) grid        */
  /* optional per-sequence storage ranges, (batch,) int32; NULL = [0,sq)/[0,sk).
   * A packed (varlen) batch passes batch strides 0 and the cu_seqlens slices.   */
  const int32_t* q_start; const int32_t* q_end;
  const int32_t* k_start; const int32_t* k_end;
  /* block-level CSR of the pattern: crow (h_pat, n_rows+1), col (h_pat, *)      */
  const int32_t* crow; const int32_t* col;
  int64_t crow_sh, col_sh;    /* head strides (0 for one shared pattern)        */
  int32_t h_pat;              /* 1, hkv or hq                                   */
  int32_t n_rows;             /* pattern rows available in crow                 */
  int32_t block_size;         /* sparse block size (power of two, 16..128)      */
  int32_t causal;
  int32_t row_mode;           /* BSA_ROWS_BY_*                                  */
  int32_t dtype;              /* BSA_F16 / BSA_BF16 / BSA_F32                   */
  int32_t impl;               /* BSA_IMPL_*                                     */
  float sm_scale;
  /* Patterns with 16- or 32-token blocks on the tensor-core forward, and on the tensor-core
   * backward when bsa_bwd_params.ds_ws is given (BSA_IMPL_SM100 / AUTO only): crow/col describe the pattern coarsened to block_size = 64, fine_block is
   * the pattern's own block size and col_bits holds, for every entry of col, one bit per
   * (sub-row a, sub-column b) pair of the 64 x 64 block, bit a * (64 / fine_block) + b.
   * 0 / NULL = the pattern's blocks are the kernel's.  The reference runs such patterns
   * through merged "micro_M" layouts (dkernel/utils.py:262-310).                       */
  const int32_t* col_bits;
  int64_t col_bits_sh;
  int32_t fine_block;
  /* Optional: 4 bytes of device memory holding 0 when the launch starts, used by this launch
   * alone (the caller zeroes them on the launch's stream, e.g. a memset node in a graph).
   * The persistent CTAs of the tensor-core forward then draw their tiles from this counter
   * as they go instead of following a fixed assignment; the outputs are the same bit for
   * bit.  NULL = fixed assignment.  No reference counterpart (Triton's grid is scheduled by
   * the hardware).                                                                       */
  int32_t* tile_counter;
} bsa_fwd_params;

int bsa_fwd(const bsa_fwd_params* p, void* stream);

/* 1 if the tcgen05 kernel serves these parameters, 0 if the generic kernel
 * does, negative on invalid parameters. */
int bsa_fwd_uses_sm100(const bsa_fwd_params* p);

/* NULL if the tcgen05 kernel serves these parameters, else the reason why
 * bsa_fwd with BSA_IMPL_AUTO would run them on the (much slower) CUDA-core
 * kernel, as static text (or the validation error).  Lets a host make the
 * fall-back visible; the reference has one kernel family and no such case. */
const char* bsa_fwd_why_not_sm100(const bsa_fwd_params* p);

/* ---------------------------------------------------------------------------
 * Attention backward.  Replaces _bwd_preprocess + _sparse_bwd_kernel
 * (dkernel/ops/sparse_attn_bwd.py:781-788, :811-850).  dQ walks the CSR, dK/dV
 * walk the CSC; every gradient tile is written once (no atomics).
 * ------------------------------------------------------------------------- */
typedef struct {
  bsa_fwd_params f;           /* same problem description; f.o = forward output,
                                 f.lse = forward LSE (required)                 */
  const void* d_o;            /* dO, strides do_*                               */
  const float* d_lse;         /* optional gradient w.r.t. LSE, strides as f.lse */
  int64_t do_sb, do_ss, do_sh;
  void* dq; void* dk; void* dv;
  int64_t dq_sb, dq_ss, dq_sh;
  int64_t dk_sb, dk_ss, dk_sh;
  int64_t dv_sb, dv_ss, dv_sh;
  const int32_t* ccol; const int32_t* row;   /* CSC of the pattern              */
  int64_t ccol_sh, row_sh;
  int32_t n_cols;             /* pattern columns available in ccol              */
  float* delta;               /* fp32 workspace of 2 * batch * hq * (sq rounded up to a
                                 multiple of 64) elements, 16-byte aligned          */
  /* Optional: which two kv blocks share a dK/dV tile of the tensor-core kernel (it computes
   * 128 kv rows at a time and walks the union of the two blocks' CSC columns, so blocks with
   * similar columns should be paired).  int32 (pairs heads, n_pairs, 2), -1 = no partner;
   * every kv block of a head appears exactly once; one table per kv head (kv_pairs_sh =
   * elements between heads) or one for all (kv_pairs_sh = 0).  NULL: blocks 2i and 2i+1. */
  const int32_t* kv_pairs;
  int64_t kv_pairs_sh;
  int32_t n_pairs;
  /* Optional dS hand-over (tensor-core kernels only; the CUDA-core kernels ignore it).  With
   * ds_ws != NULL the dK/dV kernel also stores the dS^T tile (64 x 64 elements of the input
   * dtype) of every attended block, and dQ is computed as dQ += dS K from those tiles instead
   * of recomputing S and dP: five products per attended block instead of seven (the reference's
   * one backward kernel also computes S and dP once, sparse_attn_bwd.py:86-170).
   *   ds_ws: batch * hq * ds_tiles_per_head tiles of 8192 bytes, 128-byte aligned; its contents
   *          need not be initialised and are scratch afterwards;
   *   ds_tiles_per_head: at least the number of attended blocks of any pattern head
   *          (crow[h][n_rows]);
   *   csc_csr: int32, shape and head stride of `row`: for the CSC entry at a position, the
   *          position of the same block in `col` (the CSR).                                  */
  void* ds_ws;
  int64_t ds_tiles_per_head;
  const int32_t* csc_csr;
} bsa_bwd_params;

int bsa_bwd(const bsa_bwd_params* p, void* stream);

/* ---------------------------------------------------------------------------
 * Decode: one query token per sequence against contiguous (un-paged) K/V.
 * Replaces the q_len == 1 launches of _fwd_kernel_batch_inference
 * (dkernel/ops/sparse_attn_inference.py:83-88, :141) and the sliced-crow decode
 * of _forward (dkernel/ops/sparse_attn_fwd.py:435-440).  Split-KV: every
 * (sequence, kv head, split) is one CTA; partial (O, m, l) go to the workspace
 * and are merged by a second kernel.
 * ------------------------------------------------------------------------- */
typedef struct {
  const void* q;              /* (batch, hq, d), strides q_sb, q_sh             */
  const void* k; const void* v;
  void* o; float* lse;        /* o like q; lse (batch, hq) or NULL.  o = NULL: leave the
                                 per-split partials unmerged in ws (fp32 o (batch, hq,
                                 splits, d) normalised per split, then lse (batch, hq,
                                 splits)); splits = bsa_decode_workspace_bytes(p) /
                                 (4 * batch * hq * (d + 1)), at least 1               */
  int64_t q_sb, q_sh;
  int64_t k_sb, k_ss, k_sh;
  int64_t v_sb, v_ss, v_sh;
  int64_t o_sb, o_sh;
  int64_t lse_sb, lse_sh;
  int32_t batch, hq, hkv, d, sk;
  const int32_t* k_start;     /* (batch,) first stored token, NULL = 0          */
  const int32_t* k_end;       /* (batch,) one past the last stored token, NULL = sk */
  /* KV sharding: the stored tokens of sequence b are positions
   * [k_pos0[b], k_pos0[b] + k_end[b]-k_start[b]) of a sequence whose full
   * length is k_total[b].  NULL = not sharded (pos0 = 0, total = stored).      */
  const int32_t* k_pos0; const int32_t* k_total;
  const int32_t* crow; const int32_t* col;
  int64_t crow_sh, col_sh;
  int32_t h_pat, n_rows, block_size;
  int32_t heads_per_cta;      /* q heads of one kv group handled together;
                                 they must share one pattern row (1 = safe)     */
  int32_t blocks_per_split;   /* attended blocks per CTA; <= 0: the library picks 4..16 */
  int32_t max_row_nnz;        /* longest pattern row: bounds the split count    */
  int32_t dtype;
  float sm_scale;
  float* ws;                  /* workspace, bsa_decode_workspace_bytes()        */
  /* Block-cyclic KV shard (k_blk_mod = W > 1): the stored tokens of sequence b are
   * the blocks c with c % W == k_blk_rem of a sequence of k_total[b] tokens, back
   * to back (block c is local block c / W; k_pos0 is ignored).  A local window of
   * consecutive blocks then spreads evenly over the W shards.  0 or 1 = off.   */
  int32_t k_blk_mod, k_blk_rem;
  /* 8-bit K/V cache (the reference lists "FP8 K/V" as future work, README.md:245-247):
   * kv_dtype = BSA_F8E4M3 makes k and v e4m3 tensors (strides in 1-byte elements) that
   * stand for k * k_scale and v * v_scale (per-tensor scales); q, o and the arithmetic
   * stay in `dtype`.  The kernel converts the stored bytes exactly, so the result equals
   * attention over the de-quantised cache.  0 = K/V have q's type.                     */
  int32_t kv_dtype;
  float k_scale, v_scale;
} bsa_decode_params;

size_t bsa_decode_workspace_bytes(const bsa_decode_params* p);
int bsa_decode(const bsa_decode_params* p, void* stream);

/* ---------------------------------------------------------------------------
 * bsa_decode for callers that cannot allocate.  No counterpart in the reference.
 *
 * bsa_decode needs a caller-provided workspace for its split-KV partials.  Some
 * callers have none to give: a serving runtime whose device-memory budget is
 * entirely committed to the KV cache, a plugin living inside a process whose
 * allocator it may not call, a thin language binding that can only forward the
 * tensors it received.  This variant takes the same parameters, ignores p->ws
 * and keeps the partials in a fixed array inside the library image
 * (bsa_decode_static_capacity() bytes, currently 8 MiB, resident on every GPU
 * that loads the library until the process exits).  It calls no cudaMalloc,
 * cudaFree or allocating library routine; inputs and outputs are still the
 * caller's.
 *
 *  - Limit: bsa_decode_workspace_bytes(p) must not exceed the capacity, else
 *    BSA_E_TOOBIG is returned and nothing is launched (lower batch x heads or
 *    raise blocks_per_split, or use bsa_decode).
 *  - The first call on a device looks up the array's device address (once per
 *    device, with that device current); make that first call outside any
 *    stream capture.
 *  - All calls share the one array and it keeps whatever the last call left in
 *    it.  Nothing in it has to start at zero: every slot a launch reads is
 *    written by the same launch first.  Two calls that overlap on the GPU (two
 *    streams, or two host threads on one device) race on it: serialise them.
 * ------------------------------------------------------------------------- */
int bsa_decode_static(const bsa_decode_params* p, void* stream);
size_t bsa_decode_static_capacity(void);

/* ---------------------------------------------------------------------------
 * Merge of attention partials over key/value partitions.  Replaces the eager
 * torch ops of combine_attn_partitions (dkernel/interface.py:319-324).
 * o_parts: (P, rows, d) with stride part_stride_o between partitions and
 * row_stride_o between rows; lse_parts: (P, rows) with strides part_stride_lse
 * and row_stride_lse.  Writes o (rows, d) and, if non-NULL, the merged lse
 * (rows, contiguous).  Partitions with LSE = -inf contribute nothing; a row
 * whose partitions are all -inf gives o = 0, lse = -inf.
 * ------------------------------------------------------------------------- */
int bsa_merge_partials(const void* o_parts, const float* lse_parts, int32_t P,
                       int64_t rows, int32_t d, int64_t part_stride_o,
                       int64_t row_stride_o, int64_t part_stride_lse,
                       int64_t row_stride_lse, void* o, int64_t o_row_stride,
                       float* lse, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------
 * KV-sharded decode on one node: exchange of the ranks' partial (O, LSE) rows
 * over peer memory and their merge, in one kernel per rank.  Replaces "gather
 * the partitions, then combine_attn_partitions" (dkernel/interface.py:303-324,
 * README "KV partition") and needs no collective library.
 *
 * Every rank allocates an exchange buffer of bsa_xchg_buffer_bytes() bytes,
 * zero-filled once, 256-byte aligned, and maps the buffers of all ranks (CUDA
 * IPC, or torch symmetric memory): xbuf[w] is rank w's buffer as addressed by
 * THIS process; xbuf[rank] is the local one.  Per step every rank calls
 * bsa_xchg_merge once with its partial rows (stage_o (rows, d) 16-bit
 * contiguous, stage_lse (rows) fp32; or the unmerged split partials, see the
 * struct): the kernel stores them into every rank's
 * buffer (remote stores only; nothing is loaded from peer memory) as 8-byte
 * words that carry the step number beside their payload, waits -- bounded, see
 * bsa_wait_status, code 601 -- until the words of all ranks in the local buffer
 * show the current step and writes the merged out (rows, d) and out_lse (rows,
 * or NULL).  All ranks must make the same sequence of calls with
 * the same (world, rows, d); the step counter lives in the buffer, so a captured
 * CUDA graph of the call can be replayed.  Limits: world <= 8, d % 8 == 0.
 * ------------------------------------------------------------------------- */
typedef struct {
  const void* stage_o; const float* stage_lse;
  void* out; float* out_lse;
  void* xbuf[8];
  int64_t rows;
  int32_t world, rank, d, dtype;
  /* Alternative input (stage_o = NULL): the unmerged split-KV partials a bsa_decode call with
   * o = NULL left in its workspace, fp32 (rows, nsplit, d) and (rows, nsplit).  The kernel merges
   * the splits itself, which saves the split-merge launch; it may then be enqueued right behind
   * that bsa_decode call on the same stream (it is launched as its programmatic dependent). */
  const float* part_o; const float* part_lse;
  int32_t nsplit;
} bsa_xchg_params;

size_t bsa_xchg_buffer_bytes(int32_t world, int64_t rows, int32_t d);
int bsa_xchg_merge(const bsa_xchg_params* p, void* stream);

/* ---------------------------------------------------------------------------
 * Device-side waits (on TMA / tensor-core completion barriers) are bounded.  A
 * wait that gives up records a non-zero code in a device status word and the
 * kernels of the library become no-ops until it is cleared.  This call
 * synchronises the device, copies the word to *status and clears it when
 * `reset` is non-zero.  0 = every wait completed.  No counterpart in the
 * reference (Triton kernels have no such waits).
 * ------------------------------------------------------------------------- */
int bsa_wait_status(int32_t* status, int32_t reset);

/* Optional host-visible copy of that status word for the current device: the
 * first wait that gives up also stores its code in *host_word, which must be
 * page-locked host memory the device can address (cudaHostAlloc / a pinned
 * torch tensor; the caller owns it and keeps it alive).  A host can then notice
 * a failed wait by reading the word, without synchronising.  NULL removes the
 * registration; bsa_wait_status(reset) also clears the word.  No counterpart in
 * the reference. */
int bsa_set_wait_status_mirror(int32_t* host_word);

/* Test hook: enqueues one tiny kernel that waits (at most limit_us
 * microseconds, 1..100000) on a barrier nothing ever arrives at, so that the
 * give-up path above can be observed: afterwards bsa_wait_status reports code
 * 900 and launches are no-ops until it is reset.  Nothing faults or hangs.  No
 * counterpart in the reference. */
int bsa_selftest_wait_timeout(uint32_t limit_us, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BSA_B200_H_ */
