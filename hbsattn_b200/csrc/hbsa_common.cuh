// Shared declarations of the hbsattn_b200 CUDA sources (not part of the public C ABI).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/hbsattn_b200.h"

namespace hbsa {

constexpr int kHistBins = 1024;      // work items are bucketed by min(active k-blocks, kHistBins-1)
constexpr int kStatusWords = 16;

// Carved out of the caller's workspace by make_workspace(); every pointer is a device pointer.
struct Workspace {
  int32_t* status;       // [kStatusWords]  word 0: HBSA_STATUS_*, word 1..: detail
  int32_t* cnq;          // [batch+1] first q-block of every sample
  int32_t* cnk;          // [batch+1] first k-block of every sample
  int32_t* qb2b;         // [num_q_block] sample of every q-block
  int32_t* counts;       // [nhead_k*num_q_block] active k-blocks per (kv-head, q-block) row
  int32_t* order;        // [nhead_k*num_q_block] rows sorted by descending count (bucketed)
  int32_t* hist;         // [kHistBins]
  int32_t* bin_start;    // [kHistBins]
  int32_t* bin_cursor;   // [kHistBins]
};

size_t workspace_bytes(int nhead_k, int num_q_block, int num_k_block, int batch);
Workspace make_workspace(void* base, int nhead_k, int num_q_block, int num_k_block, int batch);

// Problem description handed to every kernel (by value).
struct Problem {
  const int32_t* cu_q;
  const int32_t* cu_k;
  const uint8_t* mask;
  int64_t mask_s0, mask_s1, mask_s2;   // bytes
  int batch, nhead_q, nhead_k, group;  // group = nhead_q / nhead_k
  int headdim;
  int num_q_block, num_k_block, qbs, kbs;
  int causal;
  float scale;                          // softmax scale (natural-log domain)
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

// printf-style setter of the text hbsa_last_error() returns on the calling thread.
void set_last_error(const char* fmt, ...);

// Launchers (each enqueues on `stream` and returns the cudaError_t of the launch).
cudaError_t launch_calculate_blocks(const int32_t* cu_seqlen, int batch, int block_size, int capacity,
                                    int32_t* cu_block, int32_t* block_to_batch, int32_t* cu_num_block,
                                    cudaStream_t stream);
cudaError_t launch_schedule(const Problem& p, const Workspace& ws, uint8_t* decisions, bool need_order,
                            cudaStream_t stream);
cudaError_t launch_forward_generic(const Problem& p, const Workspace& ws, const hbsa_forward_args& a,
                                   cudaStream_t stream);
// Returns nullptr when eligible, else a static string saying why not.
const char* sm100_ineligible_reason(const hbsa_forward_args& a, float scale);
// err_text receives a message when a negative HBSA_ERR_* is returned.
int launch_forward_sm100(const Problem& p, const Workspace& ws, const hbsa_forward_args& a,
                         cudaStream_t stream, const char** err_text);

}  // namespace hbsa
