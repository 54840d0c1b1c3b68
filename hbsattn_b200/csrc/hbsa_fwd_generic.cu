// Generic CUDA-core forward: any dtype (bf16 / fp16 / fp32), any headdim <= 256, any strides,
// any softmax scale.  It covers the corners of the reference's test grid that the tensor-core
// kernel does not take (test/test_accuracy.py:24,28: fp32 inputs, headdim 18) and is the
// second, independently written implementation the tensor-core kernel is cross-checked against.
//
// One CTA = 32 query rows of one (q-block, q-head); four threads share a row and split the
// head dimension (thread s owns dims s, s+4, s+8, ...).  K/V tiles of the active k-blocks are
// staged in shared memory as fp32; scores, online softmax and the output accumulate in fp32
// registers (the arithmetic of fwd_triton_fix_tile_size.py:157-192 without the bf16 rounding of P).
#include "hbsa_common.cuh"

namespace hbsa {

template <typename T> __device__ __forceinline__ float load_f(const T* p);
template <> __device__ __forceinline__ float load_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_f<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void store_f(T* p, float x);
template <> __device__ __forceinline__ void store_f<float>(float* p, float x) { *p = x; }
template <> __device__ __forceinline__ void store_f<__half>(__half* p, float x) { *p = __float2half_rn(x); }
template <> __device__ __forceinline__ void store_f<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

struct Strides { long long q0, q1, q2, k0, k1, k2, v0, v1, v2, o0, o1, o2; };

constexpr int kRowsPerCta = 32;

template <typename T, int DQ, int KT>
__global__ void __launch_bounds__(128)
fwd_generic_kernel(Problem p, Workspace ws, const T* __restrict__ q, const T* __restrict__ k,
                   const T* __restrict__ v, T* __restrict__ o, float* __restrict__ lse, Strides st, int chunks_per_block,
                   int total_q) {
  constexpr int DPAD = DQ * 4;
  if (ws.status[0] != HBSA_STATUS_OK) {
    zero_fill_output(o, st.o0, st.o1, st.o2, total_q, p.nhead_q, p.headdim, lse);
    return;
  }
  extern __shared__ float smem[];
  float* sK = smem;                  // [KT][DPAD]
  float* sV = smem + KT * DPAD;      // [KT][DPAD]

  const int qb = blockIdx.x / chunks_per_block;
  const int chunk = blockIdx.x % chunks_per_block;
  const int hq = blockIdx.y;
  const int hk = hq / p.group;
  const RowGeom g = row_geometry(p, ws.cnq, ws.cnk, ws.qb2b, qb);
  const int row0 = g.q_begin + chunk * kRowsPerCta;
  if (row0 >= g.q_end) return;

  const int tid = threadIdx.x;
  const int r = tid >> 2, sub = tid & 3;
  const int tok = row0 + r;
  const bool valid_row = tok < g.q_end;
  const int qi = g.q_in0 + chunk * kRowsPerCta + r;
  const float scale_log2 = p.scale * 1.4426950408889634f;

  float qreg[DQ], acc[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) {
    const int d = sub + 4 * i;
    qreg[i] = (valid_row && d < p.headdim) ? load_f(q + tok * st.q0 + hq * st.q1 + d * st.q2) * scale_log2 : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  int limit_row = g.k_len - 1;
  if (p.causal) limit_row = min(limit_row, qi + g.off);

  // Active k-blocks of the row, in ascending order: bytes of the dense mask row, or the entries of the CSR row that
  // lie in the row's own sample below the causal reach.
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
          kv = load_f(k + ktok * st.k0 + hk * st.k1 + d * st.k2);
          vv = load_f(v + ktok * st.v0 + hk * st.v1 + d * st.v2);
        }
        sK[idx] = kv;
        sV[idx] = vv;
      }
      __syncthreads();
      const int key_base = blk_k0 + t0;
      for (int kk = 0; kk < nk; kk += 8) {
        float s[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float* kr = sK + (kk + u) * DPAD + sub;
          float part = 0.f;
#pragma unroll
          for (int i = 0; i < DQ; ++i) part = fmaf(qreg[i], kr[4 * i], part);
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          const bool allowed = (kk + u < nk) && (key_base + kk + u <= limit_row);
          s[u] = allowed ? part : -INFINITY;
        }
        float mx = s[0];
#pragma unroll
        for (int u = 1; u < 8; ++u) mx = fmaxf(mx, s[u]);
        const float m_new = fmaxf(m, mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = exp2f(m - m_use);
        float pr[8], psum = 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) { pr[u] = exp2f(s[u] - m_use); psum += pr[u]; }
        l = l * alpha + psum;
#pragma unroll
        for (int i = 0; i < DQ; ++i) {
          float a = acc[i] * alpha;
#pragma unroll
          for (int u = 0; u < 8; ++u) a = fmaf(pr[u], sV[(kk + u) * DPAD + sub + 4 * i], a);
          acc[i] = a;
        }
        m = m_new;
      }
    }
  }
  if (valid_row) {
    const float inv = l > 0.f ? 1.f / l : 0.f;      // rows that see no key are exact zeros
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const int d = sub + 4 * i;
      if (d < p.headdim) store_f(o + tok * st.o0 + hq * st.o1 + d * st.o2, acc[i] * inv);
    }
    // scores are kept in the log2 domain: ln sum exp = ln 2 * (m + log2 l)
    if (lse != nullptr && sub == 0) lse[(long long)tok * p.nhead_q + hq] = l > 0.f ? 0.6931471805599453f * (m + log2f(l)) : -INFINITY;
  }
}

template <typename T>
static cudaError_t launch_typed(const Problem& p, const Workspace& ws, const hbsa_forward_args& a, cudaStream_t stream) {
  Strides st{a.q_stride[0], a.q_stride[1], a.q_stride[2], a.k_stride[0], a.k_stride[1], a.k_stride[2],
             a.v_stride[0], a.v_stride[1], a.v_stride[2], a.o_stride[0], a.o_stride[1], a.o_stride[2]};
  const int cpb = (p.qbs + kRowsPerCta - 1) / kRowsPerCta;
  dim3 grid((unsigned)((long long)p.num_q_block * cpb), (unsigned)p.nhead_q);
  const T* q = static_cast<const T*>(a.q);
  const T* k = static_cast<const T*>(a.k);
  const T* v = static_cast<const T*>(a.v);
  T* o = static_cast<T*>(a.o);
#define HBSA_LAUNCH_GENERIC(DQ_, KT_)                                                                   \
  fwd_generic_kernel<T, DQ_, KT_><<<grid, 128, 2 * KT_ * DQ_ * 4 * sizeof(float), stream>>>(p, ws, q, k, v, o, a.lse, st, cpb, a.total_q)
  if (p.headdim <= 32) HBSA_LAUNCH_GENERIC(8, 32);
  else if (p.headdim <= 64) HBSA_LAUNCH_GENERIC(16, 32);
  else if (p.headdim <= 128) HBSA_LAUNCH_GENERIC(32, 32);
  else HBSA_LAUNCH_GENERIC(64, 16);
#undef HBSA_LAUNCH_GENERIC
  return cudaGetLastError();
}

cudaError_t launch_forward_generic(const Problem& p, const Workspace& ws, const hbsa_forward_args& a,
                                   cudaStream_t stream) {
  switch (a.dtype) {
    case HBSA_DTYPE_BF16: return launch_typed<__nv_bfloat16>(p, ws, a, stream);
    case HBSA_DTYPE_F16: return launch_typed<__half>(p, ws, a, stream);
    default: return launch_typed<float>(p, ws, a, stream);
  }
}

}  // namespace hbsa
