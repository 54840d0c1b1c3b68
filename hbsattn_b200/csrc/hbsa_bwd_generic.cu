// Backward of the block-sparse attention forward on the CUDA cores: dQ, dK, dV over the active block pairs.
//
// The reference has no backward (hbsattn/hbsa_interface.py:30-32 raises NotImplementedError; its README lists it
// as future work), so there is nothing to be compatible with except the mathematics of the forward it does have
// (hbsattn/reference.py:23-107).  With P = exp(scale * Q K^T - lse) on the allowed elements of the active pairs:
//     delta = rowsum(dO * O)            dV = P^T dO
//     dP = dO V^T                       dS = P * (dP - delta) * scale
//     dQ = dS K                         dK = dS^T Q
// The natural-log sum of exponentials `lse` is what the forward stores when asked to (hbsa_forward_args.lse).
//
// Same decomposition as the generic forward kernel: one CTA = 32 query rows of one (q-block, q-head), four threads
// share a row and split the head dimension; K/V tiles of the active k-blocks are staged in shared memory as fp32.
// dQ stays in the registers of the row's threads; dK and dV of a tile are summed over the CTA's rows in shared
// memory and leave with one global atomic per element and CTA into fp32 accumulators, which a last kernel casts to
// the input dtype (the q-heads of a GQA group, and all q-blocks, add into the same key rows).
#include "hbsa_common.cuh"

namespace hbsa {

namespace {

template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f(T* p, float x);
template <> __device__ __forceinline__ void st_f<float>(float* p, float x) { *p = x; }
template <> __device__ __forceinline__ void st_f<__half>(__half* p, float x) { *p = __float2half_rn(x); }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

struct BwdStrides { long long q0, q1, q2, k0, k1, k2, v0, v1, v2, o0, o1, o2, g0, g1, g2; };

constexpr int kRows = 32;

// delta[row] = sum_d dO[row, d] * O[row, d]; one warp per (token, q-head) row.
template <typename T>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta,
                                                        long long rows, int nhead_q, int headdim, BwdStrides st) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long tok = row / nhead_q, h = row % nhead_q;
  float acc = 0.f;
  for (int d = lane; d < headdim; d += 32) acc += ld_f(o + tok * st.o0 + h * st.o1 + d * st.o2) * ld_f(d_o + tok * st.g0 + h * st.g1 + d * st.g2);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[row] = acc;
}

template <typename T, int DQ, int KT>
__global__ void __launch_bounds__(128)
bwd_generic_kernel(Problem p, Workspace ws, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const T* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq,
                   float* __restrict__ dk_acc, float* __restrict__ dv_acc, BwdStrides st, int chunks_per_block, int total_q) {
  constexpr int DPAD = DQ * 4;
  if (ws.status[0] != HBSA_STATUS_OK) return;                     // the accumulators were cleared, dq is zero-filled by the caller side below
  extern __shared__ float smem[];
  float* sK = smem;                  // [KT][DPAD]
  float* sV = sK + KT * DPAD;
  float* sdK = sV + KT * DPAD;
  float* sdV = sdK + KT * DPAD;

  const int qb = blockIdx.x / chunks_per_block;
  const int chunk = blockIdx.x % chunks_per_block;
  const int hq = blockIdx.y;
  const int hk = hq / p.group;
  const RowGeom g = row_geometry(p, ws.cnq, ws.cnk, ws.qb2b, qb);
  const int row0 = g.q_begin + chunk * kRows;
  if (row0 >= g.q_end) return;

  const int tid = threadIdx.x;
  const int r = tid >> 2, sub = tid & 3;
  const int tok = row0 + r;
  const bool valid_row = tok < g.q_end;
  const int qi = g.q_in0 + chunk * kRows + r;
  const float scale_log2 = p.scale * 1.4426950408889634f;

  float qreg[DQ], greg[DQ], acc[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) {
    const int d = sub + 4 * i;
    const bool in = valid_row && d < p.headdim;
    qreg[i] = in ? ld_f(q + tok * st.q0 + hq * st.q1 + d * st.q2) : 0.f;
    greg[i] = in ? ld_f(d_o + tok * st.g0 + hq * st.g1 + d * st.g2) : 0.f;
    acc[i] = 0.f;
  }
  // rows that saw no key have lse = -inf: every P of theirs is zero
  const float lse_row = valid_row ? lse[(long long)tok * p.nhead_q + hq] : -INFINITY;
  const bool live = valid_row && lse_row > -INFINITY;
  const float lse2 = live ? lse_row * 1.4426950408889634f : 0.f;
  const float delta_row = live ? delta[(long long)tok * p.nhead_q + hq] : 0.f;
  int limit_row = g.k_len - 1;
  if (p.causal) limit_row = min(limit_row, qi + g.off);

  const bool csr = p.csr_ptr != nullptr;
  const uint8_t* mrow = csr ? nullptr : p.mask + hk * p.mask_s0 + qb * p.mask_s1;
  int e_begin = 0, n_src = g.n_reach;
  if (csr) {
    const long long row = (long long)hk * p.num_q_block + qb;
    const int e0 = p.csr_ptr[row], e1 = p.csr_ptr[row + 1];
    e_begin = lower_bound_i32(p.csr_idx, e0, e1, g.kb0);
    n_src = lower_bound_i32(p.csr_idx, e_begin, e1, g.kb0 + g.n_reach) - e_begin;
  }
  for (int e = 0; e < n_src; ++e) {
    int j = e;
    if (csr) j = p.csr_idx[e_begin + e] - g.kb0;
    else if (mrow[(long long)(g.kb0 + j) * p.mask_s2] == 0) continue;  // uniform over the CTA
    const int blk_k0 = j * p.kbs;
    const int blk_len = min(p.kbs, g.k_len - blk_k0);
    for (int t0 = 0; t0 < blk_len; t0 += KT) {
      const int nk = min(KT, blk_len - t0);
      __syncthreads();
      for (int idx = tid; idx < KT * DPAD; idx += 128) {
        const int key = idx / DPAD, d = idx % DPAD;
        float kv = 0.f, vv = 0.f;
        if (key < nk && d < p.headdim) {
          const long long ktok = g.k_begin + blk_k0 + t0 + key;
          kv = ld_f(k + ktok * st.k0 + hk * st.k1 + d * st.k2);
          vv = ld_f(v + ktok * st.v0 + hk * st.v1 + d * st.v2);
        }
        sK[idx] = kv;
        sV[idx] = vv;
        sdK[idx] = 0.f;
        sdV[idx] = 0.f;
      }
      __syncthreads();
      const int key_base = blk_k0 + t0;
      for (int kk = 0; kk < nk; ++kk) {
        const float* kr = sK + kk * DPAD + sub;
        const float* vr = sV + kk * DPAD + sub;
        float s = 0.f, dp = 0.f;
#pragma unroll
        for (int i = 0; i < DQ; ++i) {
          s = fmaf(qreg[i], kr[4 * i], s);
          dp = fmaf(greg[i], vr[4 * i], dp);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        dp += __shfl_xor_sync(0xffffffffu, dp, 1);
        dp += __shfl_xor_sync(0xffffffffu, dp, 2);
        const bool allowed = live && (key_base + kk <= limit_row);
        const float pr = allowed ? exp2f(s * scale_log2 - lse2) : 0.f;
        const float ds = pr * (dp - delta_row) * p.scale;
        if (pr != 0.f) {
          float* dkr = sdK + kk * DPAD + sub;
          float* dvr = sdV + kk * DPAD + sub;
#pragma unroll
          for (int i = 0; i < DQ; ++i) {
            acc[i] = fmaf(ds, kr[4 * i], acc[i]);
            atomicAdd(dkr + 4 * i, ds * qreg[i]);
            atomicAdd(dvr + 4 * i, pr * greg[i]);
          }
        }
      }
      __syncthreads();
      for (int idx = tid; idx < KT * DPAD; idx += 128) {
        const int key = idx / DPAD, d = idx % DPAD;
        if (key < nk && d < p.headdim) {
          const long long ktok = g.k_begin + blk_k0 + t0 + key;
          const long long off = (ktok * p.nhead_k + hk) * p.headdim + d;
          const float a = sdK[idx], b = sdV[idx];
          if (a != 0.f) atomicAdd(dk_acc + off, a);
          if (b != 0.f) atomicAdd(dv_acc + off, b);
        }
      }
    }
  }
  if (valid_row) {
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const int d = sub + 4 * i;
      if (d < p.headdim) st_f(dq + ((long long)tok * p.nhead_q + hq) * p.headdim + d, acc[i]);
    }
  }
}

template <typename T>
__global__ void bwd_cast_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) st_f(dst + i, src[i]);
}

template <typename T>
cudaError_t launch_typed(const Problem& p, const Workspace& ws, const hbsa_backward_args& b, cudaStream_t stream) {
  const hbsa_forward_args& a = b.fwd;
  BwdStrides st{a.q_stride[0], a.q_stride[1], a.q_stride[2], a.k_stride[0], a.k_stride[1], a.k_stride[2],
                a.v_stride[0], a.v_stride[1], a.v_stride[2], a.o_stride[0], a.o_stride[1], a.o_stride[2],
                b.do_stride[0], b.do_stride[1], b.do_stride[2]};
  const long long q_rows = (long long)a.total_q * a.nhead_q;
  const long long kv_elems = (long long)a.total_k * a.nhead_k * a.headdim;
  float* delta = static_cast<float*>(b.grad_workspace);
  float* dk_acc = delta + ((q_rows + 63) / 64) * 64;
  float* dv_acc = dk_acc + kv_elems;
  cudaError_t e = cudaMemsetAsync(dk_acc, 0, 2 * (size_t)kv_elems * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  // rows of q-blocks the kernel never visits (none in a consistent problem) and the error-status path leave zeros
  e = cudaMemsetAsync(b.dq, 0, (size_t)q_rows * a.headdim * sizeof(T), stream);
  if (e != cudaSuccess) return e;
  const T* q = static_cast<const T*>(a.q);
  const T* k = static_cast<const T*>(a.k);
  const T* v = static_cast<const T*>(a.v);
  const T* o = static_cast<const T*>(a.o);
  const T* d_o = static_cast<const T*>(b.d_o);
  bwd_delta_kernel<T><<<(unsigned)((q_rows + 7) / 8), 256, 0, stream>>>(o, d_o, delta, q_rows, a.nhead_q, a.headdim, st);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const int cpb = (p.qbs + kRows - 1) / kRows;
  dim3 grid((unsigned)((long long)p.num_q_block * cpb), (unsigned)p.nhead_q);
#define HBSA_LAUNCH_BWD(DQ_, KT_)                                                                                         \
  do {                                                                                                                   \
    const size_t smem = 4u * KT_ * DQ_ * 4 * sizeof(float);                                                              \
    e = cudaFuncSetAttribute(bwd_generic_kernel<T, DQ_, KT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    if (e == cudaSuccess) {                                                                                              \
      bwd_generic_kernel<T, DQ_, KT_><<<grid, 128, smem, stream>>>(p, ws, q, k, v, d_o, a.lse, delta, static_cast<T*>(b.dq), \
                                                                   dk_acc, dv_acc, st, cpb, a.total_q);                  \
      e = cudaGetLastError();                                                                                            \
    }                                                                                                                    \
  } while (0)
  if (p.headdim <= 32) HBSA_LAUNCH_BWD(8, 32);
  else if (p.headdim <= 64) HBSA_LAUNCH_BWD(16, 32);
  else if (p.headdim <= 128) HBSA_LAUNCH_BWD(32, 32);
  else HBSA_LAUNCH_BWD(64, 16);
#undef HBSA_LAUNCH_BWD
  if (e != cudaSuccess) return e;
  const unsigned blocks = (unsigned)((kv_elems + 255) / 256);
  bwd_cast_kernel<T><<<blocks, 256, 0, stream>>>(dk_acc, static_cast<T*>(b.dk), kv_elems);
  bwd_cast_kernel<T><<<blocks, 256, 0, stream>>>(dv_acc, static_cast<T*>(b.dv), kv_elems);
  return cudaGetLastError();
}

}  // namespace

size_t backward_workspace_bytes(long long total_q, long long total_k, int nhead_q, int nhead_k, int headdim) {
  const long long q_rows = total_q * nhead_q;
  return (size_t)(((q_rows + 63) / 64) * 64 + 2 * total_k * nhead_k * headdim) * sizeof(float);
}

cudaError_t launch_backward_generic(const Problem& p, const Workspace& ws, const hbsa_backward_args& b, cudaStream_t stream) {
  switch (b.fwd.dtype) {
    case HBSA_DTYPE_BF16: return launch_typed<__nv_bfloat16>(p, ws, b, stream);
    case HBSA_DTYPE_F16: return launch_typed<__half>(p, ws, b, stream);
    default: return launch_typed<float>(p, ws, b, stream);
  }
}

}  // namespace hbsa
