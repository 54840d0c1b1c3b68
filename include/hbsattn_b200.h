/*
 * hbsattn_b200 - C ABI of the B200 (sm_100a) heterogeneous block-sparse attention forward.
 *
 * Every entry point takes plain device pointers, sizes and element strides; no torch
 * types cross this boundary.  All work is enqueued on the CUDA stream passed as the
 * last argument (a cudaStream_t cast to void*; NULL = the legacy default stream) of the
 * device that is current when the call is made.  No entry point synchronises the
 * stream except hbsa_read_status().
 *
 * Return value of every int function: 0 = enqueued; negative = the arguments were
 * rejected before any launch (text in hbsa_last_error()); positive = a CUDA runtime
 * error code observed while launching.
 */
#ifndef HBSATTN_B200_H_
#define HBSATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HBSA_ABI_VERSION 4

/* Element type of q, k, v and o. */
enum { HBSA_DTYPE_BF16 = 0, HBSA_DTYPE_F16 = 1, HBSA_DTYPE_F32 = 2 };

/* Kernel family. AUTO picks the tcgen05 kernel whenever the problem is eligible
 * (bf16/fp16, headdim a multiple of 8 from 16 to 256, unit stride along headdim, 16-byte aligned rows,
 * softmax_scale > 0) and the generic CUDA-core kernel otherwise.  Forcing SM100 on an
 * ineligible problem is an argument error.  Both families are CUDA; there is no CPU path. */
enum { HBSA_IMPL_AUTO = 0, HBSA_IMPL_GENERIC = 1, HBSA_IMPL_SM100 = 2 };

/* Argument errors (negative return values). */
enum {
  HBSA_ERR_NULL = -1,        /* a required pointer is NULL                                  */
  HBSA_ERR_SHAPE = -2,       /* a size is not positive, or nhead_q % nhead_k != 0            */
  HBSA_ERR_BLOCK_SIZE = -3,  /* q/k block size is not a positive multiple of 16             */
  HBSA_ERR_DTYPE = -4,       /* unknown dtype / impl enum                                   */
  HBSA_ERR_WORKSPACE = -5,   /* workspace smaller than hbsa_workspace_bytes()               */
  HBSA_ERR_UNSUPPORTED = -6, /* HBSA_IMPL_SM100 forced on a problem it cannot run           */
  HBSA_ERR_DRIVER = -7,      /* the CUDA driver entry point for tensor maps is unavailable  */
  HBSA_ERR_STRUCT = -8       /* struct_bytes does not match this library                    */
};

/* Device-side status word (read back with hbsa_read_status). */
enum {
  HBSA_STATUS_OK = 0,
  HBSA_STATUS_BLOCK_COUNT_MISMATCH = 1, /* num_q_block/num_k_block differ from what cu_seqlens imply;
                                           no attention is computed and `o` is filled with zeros  */
  HBSA_STATUS_WAIT_LIMIT = 2            /* a bounded wait inside the attention kernel ran out       */
};

/* Library / ABI version (HBSA_ABI_VERSION of the build). */
int hbsa_version(void);

/* Text of the last argument or launch error on the calling thread. */
const char* hbsa_last_error(void);

/*
 * Block tables of a packed varlen batch, built on the device.
 * Replaces hbsattn/utils.py:7-50 (calculate_blocks), which issues ~12 torch launches.
 *
 *   cu_seqlen      int32[batch+1]  device, cumulative sequence lengths
 *   capacity       number of block entries the two block arrays can hold
 *   cu_block       int32[capacity+1] device or NULL: token offset of every block boundary
 *                  (relative to cu_seqlen[0], like the reference's cumsum at utils.py:37)
 *   block_to_batch int32[capacity]   device or NULL: sample index of every block (utils.py:39-43)
 *   cu_num_block   int32[batch+1]    device: first block index of every sample (utils.py:17-24)
 *
 * Entries beyond `capacity` are not written.  Call it once with capacity 0 to learn
 * cu_num_block[batch] (the reference also needs this one host read, utils.py:27).
 */
int hbsa_calculate_blocks(const int32_t* cu_seqlen, int batch, int block_size, int capacity,
                          int32_t* cu_block, int32_t* block_to_batch, int32_t* cu_num_block,
                          void* stream);

/* Bytes of scratch device memory hbsa_forward / hbsa_block_decisions need for a mask of
 * shape (nhead_k, num_q_block, num_k_block) and `batch` samples.  Depends on nothing else. */
size_t hbsa_workspace_bytes(int nhead_k, int num_q_block, int num_k_block, int batch);

/*
 * One forward call.  Replaces hbsattn/hbsa_interface.py:9-27 together with the launchers
 * and Triton kernels behind it (fwd_triton_auto_tile_size.py:254-310 and :76-251,
 * fwd_triton_fix_tile_size.py:216-276 and :30-212).
 *
 * Layout: q,o are [total_q, nhead_q, headdim]; k,v are [total_k, nhead_k, headdim]; packed
 * varlen, strides in ELEMENTS for (token, head, dim).  block_mask is bool bytes of shape
 * [nhead_k, num_q_block, num_k_block] over GLOBAL block indices with strides in BYTES;
 * entries that pair blocks of different samples are ignored.  cu_*_seqlens are int32[batch+1]
 * on the device.  Causal masking is aligned bottom-right when k_len != q_len.
 * use_default_scale != 0 selects headdim^-0.5 (the reference's softmax_scale=None) and ignores
 * softmax_scale.
 */
typedef struct hbsa_forward_args {
  size_t struct_bytes;            /* sizeof(hbsa_forward_args) of the caller                 */
  const void* q;
  const void* k;
  const void* v;
  void* o;
  int64_t q_stride[3];
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  const int32_t* cu_q_seqlens;
  const int32_t* cu_k_seqlens;
  const uint8_t* block_mask;
  int64_t mask_stride[3];
  int32_t total_q;
  int32_t total_k;
  int32_t nhead_q;
  int32_t nhead_k;
  int32_t headdim;
  int32_t batch;
  int32_t num_q_block;
  int32_t num_k_block;
  int32_t q_block_size;
  int32_t k_block_size;
  int32_t causal;
  int32_t use_default_scale;
  float softmax_scale;
  int32_t dtype;                  /* HBSA_DTYPE_*                                            */
  int32_t impl;                   /* HBSA_IMPL_*                                             */
  int32_t reserved;
  void* workspace;                /* >= hbsa_workspace_bytes(...) bytes, 256-byte aligned    */
  size_t workspace_bytes;
  float* lse;                     /* NULL, or float32 [total_q, nhead_q] (contiguous): natural-log sum
                                     of exponentials of every row's allowed scaled scores, -inf for
                                     rows that see no key.  The reference stores log(l) without the
                                     row maximum (fwd_triton_auto_tile_size.py:249) and never returns
                                     it; this is the value a backward pass needs.                */
  const int32_t* csr_row_ptr;     /* NULL, or the block mask in CSR form (block_mask is then ignored and may be
                                     NULL): int32 [nhead_k * num_q_block + 1], row (hk, qb) owns the entries
                                     csr_col_idx[csr_row_ptr[hk * num_q_block + qb] .. csr_row_ptr[.. + 1])   */
  const int32_t* csr_col_idx;     /* int32 [nnz]: GLOBAL k-block indices of the active pairs, ascending inside
                                     every row; entries that pair blocks of different samples are ignored.
                                     The reference has no such input: its callers cache calculate_blocks
                                     outputs by hand (test/test_speedup.py:100-102,152) and the kernels poll
                                     every mask byte of the sample (fwd_triton_fix_tile_size.py:117-124). */
} hbsa_forward_args;

int hbsa_forward(const hbsa_forward_args* args, void* stream);

/*
 * The two halves of hbsa_forward, for callers that reuse one mask over several calls (layers,
 * decode steps) the way the reference's callers reuse calculate_blocks outputs
 * (test/test_speedup.py:100-102,152).
 *   hbsa_build_schedule: block tables from cu_*_seqlens, active k-block count of every
 *       (kv-head, q-block) row, and one work record per row in launch order (kv-head major,
 *       samples from the longest k_len to the shortest, q-blocks of a sample from last to first)
 *       - all into `workspace` (q, k, v, o are not read and may be NULL).
 *   hbsa_attention: the attention kernel alone; `workspace` must hold the schedule built from the
 *       same cu_*_seqlens, block_mask, block sizes and causal flag.  A schedule serves any number
 *       of launches (the kernel rewinds its work cursor when it finishes); launches that share a
 *       schedule must not overlap on the GPU.
 */
int hbsa_build_schedule(const hbsa_forward_args* args, void* stream);
int hbsa_attention(const hbsa_forward_args* args, void* stream);

/*
 * The per-block valid/skip decision the forward uses, for checking and FLOP accounting.
 * Same arguments as hbsa_forward (q,k,v,o may be NULL).  Writes
 *   decisions  uint8[nhead_k * num_q_block * num_k_block] or NULL   1 = the block pair is computed
 *   counts     int32[nhead_k * num_q_block] or NULL                  active k-blocks per (kv-head, q-block)
 * (at least one of the two; the bitmap of a long-context problem can be far larger than its inputs)
 * The rule is the block-level consequence of the element mask of hbsattn/reference.py:56-89.
 */
int hbsa_block_decisions(const hbsa_forward_args* args, uint8_t* decisions, int32_t* counts,
                         void* stream);

/*
 * Backward of one forward call: dq, dk, dv over the active block pairs.  The reference has none
 * (hbsattn/hbsa_interface.py:30-32 raises NotImplementedError, README.md:159-163 lists it as future work);
 * the mathematics is that of hbsattn/reference.py:23-107 differentiated.
 *
 *   fwd      the arguments of the forward call: q, k, v, the forward's output in `o`, the forward's `lse`
 *            (required: run the forward with lse set), mask, sizes, workspace (the schedule is rebuilt in it)
 *   d_o      gradient of the output, same dtype as q, [total_q, nhead_q, headdim] with element strides do_stride
 *   dq, dk, dv   results in the dtype of q, contiguous [total_q, nhead_q, headdim] / [total_k, nhead_k, headdim]
 *   grad_workspace   >= hbsa_backward_workspace_bytes(...) bytes of device memory (fp32 accumulators), 256-byte aligned
 * CUDA-core kernels for every dtype and headdim <= 256; rows that saw no key get zero gradients.
 */
typedef struct hbsa_backward_args {
  size_t struct_bytes;            /* sizeof(hbsa_backward_args) of the caller */
  hbsa_forward_args fwd;
  const void* d_o;
  int64_t do_stride[3];
  void* dq;
  void* dk;
  void* dv;
  void* grad_workspace;
  size_t grad_workspace_bytes;
} hbsa_backward_args;

size_t hbsa_backward_workspace_bytes(int64_t total_q, int64_t total_k, int nhead_q, int nhead_k, int headdim);
int hbsa_backward(const hbsa_backward_args* args, void* stream);

/* Which kernel family hbsa_forward would run for these arguments: HBSA_IMPL_GENERIC or
 * HBSA_IMPL_SM100 (or a negative argument error). Launches nothing. */
int hbsa_select_impl(const hbsa_forward_args* args);

/* Copies the 16 device status words of `workspace` (word 0 = HBSA_STATUS_*, words 1.. = detail)
 * to status_out[0..15].  Synchronises `stream`.  For tests and debugging; the hot path never
 * calls it. */
int hbsa_read_status(const void* workspace, int32_t* status_out, void* stream);

/* Debugging aid (process-wide, not thread-safe).  Every wait inside the tensor-core attention kernel
 * gives up after `clocks` ticks of the SM clock (<= 0 restores the default of about two seconds): the
 * kernel then sets HBSA_STATUS_WAIT_LIMIT, all of its warps leave, and the call returns normally.
 * With stall_producer != 0 the kernel's loader warp publishes no work at all, so that every other
 * wait of the kernel runs out with nothing in flight - the way the give-up path is tested.
 * Applies to launches made after the call. */
void hbsa_debug_set_wait_budget(long long clocks, int stall_producer);

/* Debugging aid (process-wide, not thread-safe): while a device buffer of hbsa_debug_trace_bytes()
 * bytes is set, the first CTA of every tensor-core attention launch writes clock64() stamps of its
 * pipeline events into it (96 tiles x 32 int64 slots, then start time and SM of the first 512 CTAs).
 * NULL switches it off (the default); the kernel that runs then contains no stamp code. */
size_t hbsa_debug_trace_bytes(void);
void hbsa_debug_set_trace(void* device_buffer);

/*
 * hbsa_forward for callers that cannot allocate: identical to hbsa_forward except that the
 * scratch memory is a fixed array inside the library instead of `args->workspace` (which is
 * ignored, as is `workspace_bytes`; both may be 0).  It has no counterpart in the reference - it
 * exists for hosts that own all device memory themselves and give a plug-in only its inputs and
 * outputs (an inference server with a pre-reserved arena, an execute callback that bans
 * cudaMalloc).  The call allocates nothing, on the host side of CUDA or on the device.
 *
 *  - Limit: hbsa_workspace_bytes(nhead_k, num_q_block, num_k_block, batch) must not exceed
 *    HBSA_STATIC_SCRATCH_BYTES (about nhead_k * num_q_block <= 60k rows); larger problems
 *    return HBSA_ERR_WORKSPACE and hbsa_last_error() says how many bytes were needed.
 *  - Cost: every GPU that loads the library carries the array until the process exits.
 *  - The first call on each device looks up the array's device address.  With CUDA's lazy module
 *    loading this is also when the driver loads the library's device code and places the array,
 *    so this one call may allocate inside the driver and can fail on a GPU with no memory left:
 *    make it at start-up, outside any stream capture.  Later calls on that device allocate nothing.
 *  - All calls on a device share the array.  Each call re-initialises what it needs, so
 *    back-to-back calls on one stream are fine; calls that may overlap on the GPU race.
 *  - The device status words of the last call live in the array; read them with
 *    hbsa_static_scratch_status (hbsa_read_status needs a workspace pointer the caller does not have).
 */
#define HBSA_STATIC_SCRATCH_BYTES (4u << 20)
int hbsa_forward_static_scratch(const hbsa_forward_args* args, void* stream);

/* Copies the 16 device status words of the built-in scratch array of the current device (word 0 =
 * HBSA_STATUS_* of the last hbsa_forward_static_scratch call there, words 1.. = detail) to
 * status_out[0..15].  Synchronises `stream`; allocates nothing.  Like the entry point it serves, it
 * has no counterpart in the reference. */
int hbsa_static_scratch_status(int32_t* status_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HBSATTN_B200_H_ */
