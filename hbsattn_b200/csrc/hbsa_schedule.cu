// On-device block metadata and work schedule.
//
//  * calculate_blocks_*: the block tables of hbsattn/utils.py:7-50, built by two small kernels
//    instead of ~12 torch launches.
//  * schedule_*: from cu_seqlens and the block mask, the number of active k-blocks of every
//    (kv-head, q-block) row - the exact valid/skip decision - and an ordering of the rows by
//    descending work so that the attention grid starts with the longest rows (the reference
//    launches rows in index order, fwd_triton_fix_tile_size.py:242).
#include "hbsa_common.cuh"

namespace hbsa {

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

size_t workspace_bytes(int nhead_k, int num_q_block, int /*num_k_block*/, int batch) {
  size_t rows = (size_t)nhead_k * (size_t)num_q_block;
  size_t b = 0;
  b += align_up(kStatusWords * 4, 256);
  b += 2 * align_up((size_t)(batch + 1) * 4, 256);
  b += align_up((size_t)num_q_block * 4, 256);
  b += 2 * align_up(rows * 4, 256);
  b += 3 * align_up((size_t)kHistBins * 4, 256);
  return b;
}

Workspace make_workspace(void* base, int nhead_k, int num_q_block, int /*num_k_block*/, int batch) {
  size_t rows = (size_t)nhead_k * (size_t)num_q_block;
  char* p = static_cast<char*>(base);
  Workspace w;
  auto take = [&](size_t bytes) { char* r = p; p += align_up(bytes, 256); return reinterpret_cast<int32_t*>(r); };
  w.status = take(kStatusWords * 4);
  w.cnq = take((size_t)(batch + 1) * 4);
  w.cnk = take((size_t)(batch + 1) * 4);
  w.qb2b = take((size_t)num_q_block * 4);
  w.counts = take(rows * 4);
  w.order = take(rows * 4);
  w.hist = take((size_t)kHistBins * 4);
  w.bin_start = take((size_t)kHistBins * 4);
  w.bin_cursor = take((size_t)kHistBins * 4);
  return w;
}

// ---------------------------------------------------------------------------------------------
// Exclusive scan of per-sample block counts by one CTA.  out[0] = 0, out[b+1] = sum_{i<=b} nblk(i).
// ---------------------------------------------------------------------------------------------
__device__ void scan_num_blocks(const int32_t* __restrict__ cu, int batch, int bs, int32_t* __restrict__ out) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  if (tid == 0) { s_carry = 0; out[0] = 0; }
  __syncthreads();
  for (int base = 0; base < batch; base += blockDim.x) {
    const int b = base + tid;
    int x = 0;
    if (b < batch) {
      const int len = cu[b + 1] - cu[b];
      x = len > 0 ? (len + bs - 1) / bs : 0;
    }
    int incl = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += y;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nwarp ? s_warp[lane] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      s_warp[lane] = w;   // inclusive over warps
    }
    __syncthreads();
    const int warp_prefix = warp == 0 ? 0 : s_warp[warp - 1];
    const int carry = s_carry;
    if (b < batch) out[b + 1] = carry + warp_prefix + incl;
    __syncthreads();
    if (tid == 0) s_carry = carry + s_warp[nwarp - 1];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024) calc_num_blocks_kernel(const int32_t* __restrict__ cu, int batch, int bs,
                                                               int32_t* __restrict__ cu_num_block) {
  scan_num_blocks(cu, batch, bs, cu_num_block);
}

// Largest b with cnb[b] <= blk  (cnb is non-decreasing, cnb[0] = 0, blk < cnb[batch]).
__device__ __forceinline__ int sample_of_block(const int32_t* __restrict__ cnb, int batch, int blk) {
  int lo = 0, hi = batch;          // invariant: cnb[lo] <= blk < cnb[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cnb[mid] <= blk) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void fill_blocks_kernel(const int32_t* __restrict__ cu, int batch, int bs, int capacity,
                                   const int32_t* __restrict__ cnb, int32_t* __restrict__ cu_block,
                                   int32_t* __restrict__ block_to_batch) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int nb = min(cnb[batch], capacity);
  if (i == 0 && cu_block) cu_block[0] = 0;
  if (i >= nb) return;
  const int b = sample_of_block(cnb, batch, i);
  if (block_to_batch) block_to_batch[i] = b;
  if (cu_block) {
    const int end = min(cu[b] + (i - cnb[b] + 1) * bs, cu[b + 1]);
    cu_block[i + 1] = end - cu[0];
  }
}

cudaError_t launch_calculate_blocks(const int32_t* cu_seqlen, int batch, int block_size, int capacity,
                                    int32_t* cu_block, int32_t* block_to_batch, int32_t* cu_num_block,
                                    cudaStream_t stream) {
  calc_num_blocks_kernel<<<1, 1024, 0, stream>>>(cu_seqlen, batch, block_size, cu_num_block);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (cu_block || block_to_batch) {
    const int threads = 256;
    const int blocks = ((capacity > 0 ? capacity : 1) + threads - 1) / threads;
    fill_blocks_kernel<<<blocks, threads, 0, stream>>>(cu_seqlen, batch, block_size, capacity, cu_num_block,
                                                       cu_block, block_to_batch);
    e = cudaGetLastError();
  }
  return e;
}

// ---------------------------------------------------------------------------------------------
// Schedule
// ---------------------------------------------------------------------------------------------

// One CTA: both block-count scans, validation against the mask shape, and clearing of the
// status word and histogram of this call.
__global__ void __launch_bounds__(1024) sched_metadata_kernel(Problem p, Workspace ws) {
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) { ws.hist[i] = 0; ws.bin_cursor[i] = 0; }
  if (threadIdx.x < kStatusWords) ws.status[threadIdx.x] = 0;
  __syncthreads();
  scan_num_blocks(p.cu_q, p.batch, p.qbs, ws.cnq);
  scan_num_blocks(p.cu_k, p.batch, p.kbs, ws.cnk);
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nq = ws.cnq[p.batch], nk = ws.cnk[p.batch];
    if (nq != p.num_q_block || nk != p.num_k_block) {
      ws.status[0] = HBSA_STATUS_BLOCK_COUNT_MISMATCH;
      ws.status[1] = nq;
      ws.status[2] = nk;
    }
  }
}

__global__ void sched_qb2b_kernel(Problem p, Workspace ws) {
  if (ws.status[0] != HBSA_STATUS_OK) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.num_q_block) return;
  ws.qb2b[i] = sample_of_block(ws.cnq, p.batch, i);
}

// One warp per (kv-head, q-block) row: count the active k-blocks (mask AND same sample AND
// causal-reachable); optionally write the whole decision row.
__global__ void __launch_bounds__(256) sched_count_kernel(Problem p, Workspace ws, uint8_t* __restrict__ decisions) {
  if (ws.status[0] != HBSA_STATUS_OK) return;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)p.nhead_k * p.num_q_block;
  if (row >= rows) return;
  const int hk = (int)(row / p.num_q_block), qb = (int)(row % p.num_q_block);
  const RowGeom g = row_geometry(p, ws.cnq, ws.cnk, ws.qb2b, qb);
  const uint8_t* mrow = p.mask + hk * p.mask_s0 + qb * p.mask_s1;
  int cnt = 0;
  for (int j = lane; j < g.n_reach; j += 32) cnt += mrow[(long long)(g.kb0 + j) * p.mask_s2] != 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
  if (lane == 0) {
    ws.counts[row] = cnt;
    atomicAdd(&ws.hist[min(cnt, kHistBins - 1)], 1);
  }
  if (decisions) {
    uint8_t* drow = decisions + (size_t)row * p.num_k_block;
    for (int kb = lane; kb < p.num_k_block; kb += 32) {
      const int j = kb - g.kb0;
      const bool act = j >= 0 && j < g.n_reach && mrow[(long long)kb * p.mask_s2] != 0;
      drow[kb] = act ? 1 : 0;
    }
  }
}

// bin_start[c] = number of rows whose bin is larger than c (rows are emitted longest first).
__global__ void __launch_bounds__(kHistBins) sched_scan_kernel(Workspace ws) {
  if (ws.status[0] != HBSA_STATUS_OK) return;
  __shared__ int s[kHistBins];
  const int t = threadIdx.x;
  s[t] = ws.hist[kHistBins - 1 - t];       // reversed: index 0 is the largest bin
  __syncthreads();
  for (int d = 1; d < kHistBins; d <<= 1) {
    const int y = t >= d ? s[t - d] : 0;
    __syncthreads();
    s[t] += y;
    __syncthreads();
  }
  const int excl = t == 0 ? 0 : s[t - 1];
  ws.bin_start[kHistBins - 1 - t] = excl;
}

__global__ void sched_scatter_kernel(Problem p, Workspace ws) {
  if (ws.status[0] != HBSA_STATUS_OK) return;
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long rows = (long long)p.nhead_k * p.num_q_block;
  if (row >= rows) return;
  const int bin = min(ws.counts[row], kHistBins - 1);
  const int pos = atomicAdd(&ws.bin_cursor[bin], 1);
  ws.order[ws.bin_start[bin] + pos] = (int)row;
}

cudaError_t launch_schedule(const Problem& p, const Workspace& ws, uint8_t* decisions, bool need_order,
                            cudaStream_t stream) {
  cudaError_t e;
  sched_metadata_kernel<<<1, 1024, 0, stream>>>(p, ws);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  sched_qb2b_kernel<<<(p.num_q_block + 255) / 256, 256, 0, stream>>>(p, ws);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const long long rows = (long long)p.nhead_k * p.num_q_block;
  sched_count_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(p, ws, decisions);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  if (need_order) {
    sched_scan_kernel<<<1, kHistBins, 0, stream>>>(ws);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    sched_scatter_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, stream>>>(p, ws);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace hbsa
