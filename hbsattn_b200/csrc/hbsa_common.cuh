// Shared declarations of the hbsattn_b200 CUDA sources (not part of the public C ABI).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <math.h>

#include "../../include/hbsattn_b200.h"

namespace hbsa {

constexpr int kStatusWords = 16;
constexpr int kItemWords = 16;       // int32 words of one ItemRecord

// Carved out of the caller's workspace by make_workspace(); every pointer is a device pointer.
struct Workspace {
  int32_t* status;       // [kStatusWords]  word 0: HBSA_STATUS_*, word 1..: detail
  int32_t* cnq;          // [batch+1] first q-block of every sample
  int32_t* cnk;          // [batch+1] first k-block of every sample
  int32_t* qb2b;         // [num_q_block] sample of every q-block
  int32_t* counts;       // [nhead_k*num_q_block] active k-blocks per (kv-head, q-block) row
  int32_t* items;        // [nhead_k*num_q_block][kItemWords] ItemRecord of every row, in launch order
  int32_t* cursor;       // [64] word 0: next work item of the persistent attention kernel
  int32_t* qpos;         // [batch] launch position (in q-blocks) of every sample inside a kv-head
};

// Everything the attention kernel needs to know about one (kv-head, q-block) row, written once by
// the schedule kernel so that a CTA fetches its next piece of work with a single 64-byte load.
// Launch order: kv-head major, then samples from the longest k_len to the shortest, and inside a
// sample the q-blocks from last to first (under a causal mask the longest rows come first), so the
// queue drains on short rows and the CTAs that run at the same time share the K/V of a few
// (sample, kv-head) units in L2.
struct __align__(16) ItemRecord {
  int hk, qb, q_begin, q_end;        // kv-head, q-block, token range of the q-block (global)
  int q_in0, k_begin, k_len, kb0;    // in-sample index of the first row; the sample's keys and first k-block
  int n_reach, off, n_tiles, count;  // causal-reachable k-blocks, k_len - q_len, K/V tiles to process, active blocks
  int csr_begin;                     // CSR block masks: position in col_idx of the row's first active, reachable entry
  int pad[3];
};
static_assert(sizeof(ItemRecord) == kItemWords * 4, "ItemRecord layout");

size_t workspace_bytes(int nhead_k, int num_q_block, int num_k_block, int batch);
Workspace make_workspace(void* base, int nhead_k, int num_q_block, int num_k_block, int batch);

// Problem description handed to every kernel (by value).
struct Problem {
  const int32_t* cu_q;
  const int32_t* cu_k;
  const uint8_t* mask;                 // dense block mask, or NULL when the mask is given in CSR form
  int64_t mask_s0, mask_s1, mask_s2;   // bytes
  const int32_t* csr_ptr;              // CSR block mask: [nhead_k * num_q_block + 1] row starts, or NULL
  const int32_t* csr_idx;              // [nnz] global k-block indices, ascending inside every row
  int batch, nhead_q, nhead_k, group;  // group = nhead_q / nhead_k
  int headdim;
  int num_q_block, num_k_block, qbs, kbs;
  int causal;
  float scale;                          // softmax scale (natural-log domain)
  int kv_tile;                          // rows of one K/V tile of the tensor-core kernel (0: one tile per k-block)
};

// Geometry of one (q-block, sample) pair, derived on the device from cu_seqlens only.
struct RowGeom {
  int b;            // sample
  int q_begin;      // first token of the q-block (global)
  int q_end;        // one past the last token of the q-block (global)
  int q_in0;        // in-sample index of the first row
  int k_begin;      // first key token of the sample (global)
  int k_len;        // keys in the sample
  int kb0;          // first k-block of the sample (global block index)
  int nkb;          // k-blocks in the sample
  int off;          // k_len - q_len (bottom-right causal alignment)
  int n_reach;      // k-blocks [0, n_reach) of the sample can hold a causal-valid element
};

__device__ __forceinline__ RowGeom row_geometry(const Problem& p, const int32_t* cnq, const int32_t* cnk,
                                                const int32_t* qb2b, int qb) {
  RowGeom g;
  g.b = qb2b[qb];
  const int cq0 = p.cu_q[g.b], cq1 = p.cu_q[g.b + 1];
  const int ck0 = p.cu_k[g.b], ck1 = p.cu_k[g.b + 1];
  g.q_begin = cq0 + (qb - cnq[g.b]) * p.qbs;
  g.q_end = min(g.q_begin + p.qbs, cq1);
  g.q_in0 = g.q_begin - cq0;
  g.k_begin = ck0;
  g.k_len = ck1 - ck0;
  g.kb0 = cnk[g.b];
  g.nkb = cnk[g.b + 1] - g.kb0;
  g.off = g.k_len - (cq1 - cq0);
  int reach = g.nkb;
  if (p.causal) {
    // last row of the q-block, bottom-right aligned: key index it may see at most
    const int limit = (g.q_end - 1 - cq0) + g.off;
    reach = limit < 0 ? 0 : min(g.nkb, limit / p.kbs + 1);
  }
  g.n_reach = reach;
  return g;
}

// What the attention kernels do when the schedule kernels left an error status: nothing is computed, and the
// output is filled with zeros (lse with -inf) so that a caller who does not read the status never sees
// uninitialised memory.  Called by every thread of every CTA of a one- or two-dimensional grid.
template <typename T>
__device__ __forceinline__ void zero_fill_output(T* o, long long s0, long long s1, long long s2, int total_q, int nhead_q,
                                                 int headdim, float* lse) {
  const long long n_cta = (long long)gridDim.x * gridDim.y;
  const long long cta = (long long)blockIdx.y * gridDim.x + blockIdx.x;
  const long long rows = (long long)total_q * nhead_q;
  for (long long row = cta; row < rows; row += n_cta) {
    const long long tok = row / nhead_q, h = row % nhead_q;
    for (int d = threadIdx.x; d < headdim; d += blockDim.x) o[tok * s0 + h * s1 + d * s2] = T(0.f);
    if (lse != nullptr && threadIdx.x == 0) lse[row] = -INFINITY;
  }
}

// First position in [lo, hi) of the ascending array `a` whose value is >= key (hi if there is none).
__device__ __forceinline__ int lower_bound_i32(const int32_t* __restrict__ a, int lo, int hi, int key) {
  while (lo < hi) {
    const int mid = lo + ((hi - lo) >> 1);
    if (a[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// printf-style setter of the text hbsa_last_error() returns on the calling thread.
void set_last_error(const char* fmt, ...);

// Launchers (each enqueues on `stream` and returns the cudaError_t of the launch).
cudaError_t launch_calculate_blocks(const int32_t* cu_seqlen, int batch, int block_size, int capacity,
                                    int32_t* cu_block, int32_t* block_to_batch, int32_t* cu_num_block,
                                    cudaStream_t stream);
cudaError_t launch_schedule(const Problem& p, const Workspace& ws, uint8_t* decisions, cudaStream_t stream);
// Rows of one K/V tile the tensor-core kernel uses for k blocks of `kbs` rows.
int sm100_kv_tile_rows(int kbs);
// Debugging aid: clock budget of every wait inside the tensor-core kernel (<= 0: the default), and a mode in
// which its producer warp publishes nothing, so that every other wait of the kernel runs out.
void sm100_set_wait_budget(long long clocks, int stall_producer);
// Debugging aid: clock64 stamps of the first CTA's pipeline events go to this device buffer (NULL: off).
void sm100_set_trace(long long* device_buffer);
size_t sm100_trace_bytes();
cudaError_t launch_forward_generic(const Problem& p, const Workspace& ws, const hbsa_forward_args& a,
                                   cudaStream_t stream);
size_t backward_workspace_bytes(long long total_q, long long total_k, int nhead_q, int nhead_k, int headdim);
cudaError_t launch_backward_generic(const Problem& p, const Workspace& ws, const hbsa_backward_args& b, cudaStream_t stream);
// Returns nullptr when eligible, else a static string saying why not.
const char* sm100_ineligible_reason(const hbsa_forward_args& a, float scale);
// err_text receives a message when a negative HBSA_ERR_* is returned.
int launch_forward_sm100(const Problem& p, const Workspace& ws, const hbsa_forward_args& a,
                         cudaStream_t stream, const char** err_text);

}  // namespace hbsa
