// On-device block metadata and work schedule.
//
//  * calculate_blocks_*: the block tables of hbsattn/utils.py:7-50, built by two small kernels
//    instead of ~12 torch launches.
//  * sched_*: from cu_seqlens and the block mask, the number of active k-blocks of every
//    (kv-head, q-block) row - the exact valid/skip decision - and one ItemRecord per row in the
//    order the persistent attention kernel drains them (the reference launches one program per
//    row in index order, fwd_triton_fix_tile_size.py:242).
#include "hbsa_common.cuh"

namespace hbsa {

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

size_t workspace_bytes(int nhead_k, int num_q_block, int /*num_k_block*/, int batch) {
  size_t rows = (size_t)nhead_k * (size_t)num_q_block;
  size_t b = 0;
  b += align_up(kStatusWords * 4, 256);
  b += 2 * align_up((size_t)(batch + 1) * 4, 256);
  b += align_up((size_t)num_q_block * 4, 256);
  b += align_up(rows * 4, 256);
  b += align_up(rows * kItemWords * 4, 256);
  b += align_up(64 * 4, 256);
  b += align_up((size_t)batch * 4, 256);
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
  w.items = take(rows * kItemWords * 4);
  w.cursor = take(64 * 4);
  w.qpos = take((size_t)batch * 4);
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
// status words and the work cursor of this call.
__global__ void __launch_bounds__(1024) sched_metadata_kernel(Problem p, Workspace ws) {
  if (threadIdx.x < 64) ws.cursor[threadIdx.x] = 0;
  if (threadIdx.x < kStatusWords) ws.status[threadIdx.x] = 0;
  __syncthreads();
  scan_num_blocks(p.cu_q, p.batch, p.qbs, ws.cnq);
  scan_num_blocks(p.cu_k, p.batch, p.kbs, ws.cnk);
  __syncthreads();
  // Launch position of every sample: samples sorted by descending k_len (ties by index), counted in
  // q-blocks.  Quadratic in the batch size, so very large batches keep their natural order.
  for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
    int pos = ws.cnq[b];
    if (p.batch <= 4096) {
      const int len_b = p.cu_k[b + 1] - p.cu_k[b];
      pos = 0;
      for (int o = 0; o < p.batch; ++o) {
        const int len_o = p.cu_k[o + 1] - p.cu_k[o];
        if (len_o > len_b || (len_o == len_b && o < b)) pos += ws.cnq[o + 1] - ws.cnq[o];
      }
    }
    ws.qpos[b] = pos;
  }
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
// causal-reachable); optionally write the whole decision row.  The mask is either the dense byte array
// or a CSR list of k-block indices per row.
__global__ void __launch_bounds__(256) sched_count_kernel(Problem p, Workspace ws, uint8_t* __restrict__ decisions) {
  if (ws.status[0] != HBSA_STATUS_OK) return;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)p.nhead_k * p.num_q_block;
  if (row >= rows) return;
  const int hk = (int)(row / p.num_q_block), qb = (int)(row % p.num_q_block);
  const RowGeom g = row_geometry(p, ws.cnq, ws.cnk, ws.qb2b, qb);
  const int j_last = g.nkb - 1;                 // the ragged last k-block of the sample may own fewer tiles
  int cnt = 0, csr_begin = 0;
  bool last_active = false;
  const uint8_t* mrow = nullptr;
  if (p.csr_ptr != nullptr) {
    // CSR row: ascending global k-block indices; the active ones are those of the row's own sample below the causal reach
    const int e0 = p.csr_ptr[row], e1 = p.csr_ptr[row + 1];
    csr_begin = lower_bound_i32(p.csr_idx, e0, e1, g.kb0);
    const int hi = lower_bound_i32(p.csr_idx, csr_begin, e1, g.kb0 + g.n_reach);
    cnt = hi - csr_begin;
    last_active = cnt > 0 && j_last < g.n_reach && p.csr_idx[hi - 1] == g.kb0 + j_last;
  } else {
    mrow = p.mask + hk * p.mask_s0 + qb * p.mask_s1;
    for (int j = lane; j < g.n_reach; j += 32) cnt += mrow[(long long)(g.kb0 + j) * p.mask_s2] != 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
    last_active = cnt > 0 && j_last < g.n_reach && mrow[(long long)(g.kb0 + j_last) * p.mask_s2] != 0;
  }
  if (lane == 0) {
    ws.counts[row] = cnt;
    int n_tiles = cnt;
    if (p.kv_tile > 0 && p.kv_tile < p.kbs) {
      const int n_sub = p.kbs / p.kv_tile;
      n_tiles = cnt * n_sub;
      if (last_active) {
        const int len_last = g.k_len - j_last * p.kbs;
        n_tiles -= n_sub - (len_last + p.kv_tile - 1) / p.kv_tile;
      }
    }
    ItemRecord rec;
    rec.hk = hk; rec.qb = qb; rec.q_begin = g.q_begin; rec.q_end = g.q_end;
    rec.q_in0 = g.q_in0; rec.k_begin = g.k_begin; rec.k_len = g.k_len; rec.kb0 = g.kb0;
    rec.n_reach = g.n_reach; rec.off = g.off; rec.n_tiles = n_tiles; rec.count = cnt;
    rec.csr_begin = csr_begin; rec.pad[0] = rec.pad[1] = rec.pad[2] = 0;
    // launch position: kv-head, then the sample's slot, q-blocks mirrored (last q-block of the sample first)
    const int last = ws.cnq[g.b + 1] - 1;
    const long long pos = (long long)hk * p.num_q_block + (ws.qpos[g.b] + (last - qb));
    reinterpret_cast<ItemRecord*>(ws.items)[pos] = rec;
  }
  if (decisions) {
    uint8_t* drow = decisions + (size_t)row * p.num_k_block;
    if (p.csr_ptr != nullptr) {
      for (int kb = lane; kb < p.num_k_block; kb += 32) drow[kb] = 0;
      __syncwarp();
      for (int e = csr_begin + lane; e < csr_begin + cnt; e += 32) drow[p.csr_idx[e]] = 1;
    } else {
      for (int kb = lane; kb < p.num_k_block; kb += 32) {
        const int j = kb - g.kb0;
        const bool act = j >= 0 && j < g.n_reach && mrow[(long long)kb * p.mask_s2] != 0;
        drow[kb] = act ? 1 : 0;
      }
    }
  }
}

cudaError_t launch_schedule(const Problem& p, const Workspace& ws, uint8_t* decisions, cudaStream_t stream) {
  cudaError_t e;
  sched_metadata_kernel<<<1, 1024, 0, stream>>>(p, ws);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  sched_qb2b_kernel<<<(p.num_q_block + 255) / 256, 256, 0, stream>>>(p, ws);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const long long rows = (long long)p.nhead_k * p.num_q_block;
  sched_count_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(p, ws, decisions);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  return cudaSuccess;
}

}  // namespace hbsa
