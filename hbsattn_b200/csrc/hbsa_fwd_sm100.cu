// Block-sparse attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces the two Triton kernels of the reference (fwd_triton_fix_tile_size.py:30-212,
// fwd_triton_auto_tile_size.py:76-251).  Differences of design, not of result:
//
//  * A work item is one 128-row M tile of one (kv-head, q-block): `TT = 128 / GP` tokens times
//    `GP` q-heads of the GQA group packed into the MMA M dimension, so that one K/V tile fetch
//    serves GP heads (the reference runs one program per q-head and re-reads K/V per head).
//  * Items are launched longest first (order[] from the schedule kernels), two CTAs per SM.
//  * Only mask-active k-blocks are touched: the producer warp compacts the mask row with warp
//    ballots and issues TMA loads of exactly those K/V tiles (the reference loops over all
//    k-blocks of the sample and polls the mask byte, fwd_triton_fix_tile_size.py:117-124).
//  * S = Q K^T and O += P V are tcgen05.mma instructions with fp32 accumulators in TMEM; P (in
//    the input dtype, as at fwd_triton_fix_tile_size.py:187) is written back into TMEM over S
//    and consumed as the A operand of the second MMA, so it never touches shared memory.
//  * Online softmax runs in registers, one thread per row, exp2 with the scale folded in; the
//    running output is rescaled only when a row maximum grows by more than 2^8.
//
// Warp roles (192 threads): warps 0-3 softmax + epilogue (TMEM lane quarter = warp id),
// warp 4 TMA producer, warp 5 TMEM allocator + MMA issuer.
//
// Per k-tile t the mbarriers complete exactly once, so the phase parity of tile t is t & 1:
//   k_full / v_full : TMA bytes landed            s_full : S = Q K^T done (K buffer free again)
//   p_full          : 128 rows of P written       pv_done: O += P V done (V buffer and S/P free)
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>
#include <type_traits>

#include "hbsa_common.cuh"
#include "sm100_ptx.cuh"

namespace hbsa {

namespace {

constexpr int kThreads = 192;
constexpr int kTmemCols = 256;       // S/P at columns [0,128), O at [128,128+D)
constexpr int kTmemOCol = 128;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct Sm100Params {
  Problem p;
  Workspace ws;
  void* o;
  long long o_s0, o_s1;        // elements
  int nt;                      // rows of one K/V tile (multiple of 16, <= 128)
  int n_sub;                   // K/V tiles per k-block
  int gp, gp_shift;            // q-heads packed into one M tile
  int n_head_sub;              // group / gp
  int tt;                      // tokens per M tile = 128 / gp
  int tiles_per_qblock;
  int items_per_row;           // n_head_sub * tiles_per_qblock
  float scale_log2;
  long long wait_budget;       // clock64 ticks
};

struct __align__(8) Control {
  unsigned long long q_full, k_full, v_full, s_full, p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
  int tile_k0[4];
};

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Sm100Params P) {
  using namespace ptx;
  constexpr int PANELS = D / 64;
  constexpr uint32_t Q_BYTES = 128u * D * 2u;
  constexpr uint32_t KV_BYTES_MAX = 128u * D * 2u;
  const Problem& p = P.p;

  if (P.ws.status[0] != HBSA_STATUS_OK) return;

  // ---- which item (uniform over the CTA)
  const int sorted = blockIdx.x / P.items_per_row;
  const int rem = blockIdx.x % P.items_per_row;
  const int row = P.ws.order[sorted];
  const int hk = row / p.num_q_block, qb = row % p.num_q_block;
  const int hsub = rem / P.tiles_per_qblock, qt = rem % P.tiles_per_qblock;
  const RowGeom g = row_geometry(p, P.ws.cnq, P.ws.cnk, P.ws.qb2b, qb);
  const int tile_tok0 = g.q_begin + qt * P.tt;
  if (tile_tok0 >= g.q_end) return;
  const int head0 = hk * p.group + hsub * P.gp;
  const uint8_t* mrow = p.mask + hk * p.mask_s0 + qb * p.mask_s1;
  const int count = P.ws.counts[row];
  int n_tiles = count * P.n_sub;
  if (P.n_sub > 1 && count > 0) {
    // the ragged last k-block of the sample may own fewer tiles
    const int j_last = g.nkb - 1;
    if (j_last < g.n_reach && mrow[(long long)(g.kb0 + j_last) * p.mask_s2] != 0) {
      const int len_last = g.k_len - j_last * p.kbs;
      n_tiles -= P.n_sub - (len_last + P.nt - 1) / P.nt;
    }
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  OutT* const o_base = static_cast<OutT*>(P.o);

  // Row handled by a softmax thread (warps 0-3).
  const int r_tok = tile_tok0 + (tid >> P.gp_shift);
  const int r_head = head0 + (tid & (P.gp - 1));
  const bool r_valid = tid < 128 && r_tok < g.q_end;

  if (n_tiles == 0) {
    // No active k-block: the rows are exact zeros (fwd_triton_fix_tile_size.py:189).
    if (r_valid) {
      uint4* dst = reinterpret_cast<uint4*>(o_base + r_tok * P.o_s0 + r_head * P.o_s1);
#pragma unroll
      for (int i = 0; i < D / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* const smem = smem_raw + pad;
  const uint32_t sQ = raw_addr + pad;
  const uint32_t sK = sQ + Q_BYTES;
  const uint32_t sV = sK + KV_BYTES_MAX;
  Control* const ctl = reinterpret_cast<Control*>(smem + Q_BYTES + 2 * KV_BYTES_MAX);
  const uint32_t bar_q_full = smem_u32(&ctl->q_full), bar_k_full = smem_u32(&ctl->k_full);
  const uint32_t bar_v_full = smem_u32(&ctl->v_full), bar_s_full = smem_u32(&ctl->s_full);
  const uint32_t bar_p_full = smem_u32(&ctl->p_full), bar_pv_done = smem_u32(&ctl->pv_done);
  volatile int* const abort_flag = &ctl->abort_flag;
  volatile int* const tile_k0 = ctl->tile_k0;

  if (tid == 0) {
    mbar_init(bar_q_full, 1);
    mbar_init(bar_k_full, 1);
    mbar_init(bar_v_full, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 128);
    mbar_init(bar_pv_done, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t tS = tmem_base;                 // S (fp32) and, aliased, P (16-bit pairs)
  const uint32_t tO = tmem_base + kTmemOCol;
  const long long budget = P.wait_budget;
  const uint32_t kv_tile_bytes = (uint32_t)P.nt * D * 2u;
  const uint32_t kv_panel_bytes = (uint32_t)P.nt * 128u;

  if (warp == 4) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q_full, Q_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(sQ + pn * (128u * 128u), &tm_q, bar_q_full, pn * 64, head0, tile_tok0);
    }
    int t = 0;
    bool ok = true;
    for (int base = 0; base < g.n_reach && ok; base += 32) {
      const int j = base + lane;
      const bool bit = j < g.n_reach && mrow[(long long)(g.kb0 + j) * p.mask_s2] != 0;
      uint32_t bal = __ballot_sync(0xffffffffu, bit);
      while (bal != 0 && ok) {
        const int jj = base + __ffs(bal) - 1;
        bal &= bal - 1;
        const int blk_k0 = jj * p.kbs;
        for (int sub = 0; sub < P.n_sub && ok; ++sub) {
          const int k0 = blk_k0 + sub * P.nt;
          if (k0 >= g.k_len) break;
          if (t > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_s_full, (t - 1) & 1, abort_flag, budget));
          if (!ok) break;
          if (lane == 0) {
            tile_k0[t & 3] = k0;
            __threadfence_block();
            mbar_arrive_expect_tx(bar_k_full, kv_tile_bytes);
#pragma unroll
            for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(sK + pn * kv_panel_bytes, &tm_k, bar_k_full, pn * 64, hk, g.k_begin + k0);
          }
          if (t > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_pv_done, (t - 1) & 1, abort_flag, budget));
          if (!ok) break;
          if (lane == 0) {
            mbar_arrive_expect_tx(bar_v_full, kv_tile_bytes);
#pragma unroll
            for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(sV + pn * kv_panel_bytes, &tm_v, bar_v_full, pn * 64, hk, g.k_begin + k0);
          }
          ++t;
        }
      }
    }
    if (!ok && t > 0) {
      // Gave up: let the copies already issued land before the CTA retires (bounded).
      mbar_wait_bounded(bar_k_full, (t - 1) & 1, abort_flag, budget >> 4);
    }
  } else if (warp == 5) {
    // =============================== MMA issuer ===============================
    const uint32_t idesc_qk = make_idesc(BF16, false, false, 128, P.nt);
    const uint32_t idesc_pv = make_idesc(BF16, false, true, 128, D);
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_q_full, 0, abort_flag, budget));
    for (int t = 0; t < n_tiles && ok; ++t) {
      bool w = mbar_wait_bounded(bar_k_full, t & 1, abort_flag, budget);
      if (t > 0) w = w && mbar_wait_bounded(bar_pv_done, (t - 1) & 1, abort_flag, budget);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t da = make_smem_desc(sQ + (ks >> 2) * (128u * 128u) + (ks & 3) * 32u, 16u, 1024u);
          const uint64_t db = make_smem_desc(sK + (ks >> 2) * kv_panel_bytes + (ks & 3) * 32u, 16u, 1024u);
          mma_ss(tS, da, db, idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc_commit(bar_s_full);
      }
      __syncwarp();
      w = mbar_wait_bounded(bar_v_full, t & 1, abort_flag, budget);
      w = w && mbar_wait_bounded(bar_p_full, t & 1, abort_flag, budget);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const int ksteps = P.nt >> 4;
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint64_t db = make_smem_desc(sV + ks * 2048u, kv_panel_bytes, 1024u);
          mma_ts(tO, tS + ks * 8u, db, idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(bar_pv_done);
      }
      __syncwarp();
    }
  } else {
    // =============================== softmax + epilogue ===============================
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const int qi = g.q_in0 + qt * P.tt + (tid >> P.gp_shift);          // in-sample row index
    int limit_row = g.k_len - 1;
    if (p.causal) limit_row = min(limit_row, qi + g.off);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const int nt = P.nt;
    for (int t = 0; t < n_tiles && ok; ++t) {
      // Only s_full is waited on here: k_full may already be a phase ahead (the next K tile is
      // loaded as soon as S is done), and tile_k0[] was published before the K tile of S was issued.
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_s_full, t & 1, abort_flag, budget));
      if (!ok) break;
      tc_fence_after();
      const int col_limit = limit_row - tile_k0[t & 3];                // columns <= col_limit are valid

      // ---- pass 1: row maximum of the valid columns
      float mx = -INFINITY;
      for (int c0 = 0; c0 < nt; c0 += 32) {
        if (c0 + 32 <= nt) {
          uint32_t r[32];
          tmem_ld32(tS + lane_off + c0, r);
          tmem_wait_ld();
          if (col_limit >= c0 + 31) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (c0 + i <= col_limit) ? __uint_as_float(r[i]) : -INFINITY);
          }
        } else {
          uint32_t r[16];
          tmem_ld16(tS + lane_off + c0, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) mx = fmaxf(mx, (c0 + i <= col_limit) ? __uint_as_float(r[i]) : -INFINITY);
        }
      }
      const float mx_s = mx * P.scale_log2;                              // scale > 0 keeps the order
      if (t == 0) {
        m_ref = mx_s;
      } else {
        const bool need = mx_s > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O and l move to the new reference maximum; needs O += P V of the previous tile.
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_pv_done, (t - 1) & 1, abort_flag, budget));
          if (!ok) break;
          tc_fence_after();
          const float alpha = need ? ex2_approx(m_ref - mx_s) : 1.f;
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tO + lane_off + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + lane_off + c0, r);
          }
          tmem_wait_st();
          l *= alpha;
          if (need) m_ref = mx_s;
        }
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const float neg_m = -m_use;

      // ---- pass 2: P = exp2(S * scale - m), row sum, P packed to 16 bit over S
      float sum = 0.f;
      for (int c0 = 0; c0 < nt; c0 += 32) {
        if (c0 + 32 <= nt) {
          uint32_t r[32], pk[16];
          tmem_ld32(tS + lane_off + c0, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), P.scale_log2, neg_m));
            float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), P.scale_log2, neg_m));
            if (c0 + i > col_limit) p0 = 0.f;
            if (c0 + i + 1 > col_limit) p1 = 0.f;
            sum += p0 + p1;
            pk[i >> 1] = pack2<BF16>(p0, p1);
          }
          tmem_st16(tS + lane_off + (c0 >> 1), pk);
        } else {
          uint32_t r[16], pk[8];
          tmem_ld16(tS + lane_off + c0, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), P.scale_log2, neg_m));
            float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), P.scale_log2, neg_m));
            if (c0 + i > col_limit) p0 = 0.f;
            if (c0 + i + 1 > col_limit) p1 = 0.f;
            sum += p0 + p1;
            pk[i >> 1] = pack2<BF16>(p0, p1);
          }
          tmem_st8(tS + lane_off + (c0 >> 1), pk);
        }
      }
      l += sum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full);
    }

    // ---- epilogue: O / l -> global, 16-byte stores, rows past the q-block end are dropped
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_pv_done, (n_tiles - 1) & 1, abort_flag, budget));
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      OutT* const orow = o_base + r_tok * P.o_s0 + r_head * P.o_s1;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tO + lane_off + c0, r);
        tmem_wait_ld();
        if (r_valid) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a = l > 0.f ? __uint_as_float(r[i]) * inv : 0.f;
            const float b = l > 0.f ? __uint_as_float(r[i + 1]) * inv : 0.f;
            pk[i >> 1] = pack2<BF16>(a, b);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        }
      }
    }
  }

  // ---- teardown: every thread gets here (all waits are bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag) {
    atomicExch(&P.ws.status[0], HBSA_STATUS_WAIT_LIMIT);
    P.ws.status[3] = (int)blockIdx.x;
  }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 3-D map over a [tokens, heads, headdim] tensor: dims (headdim, heads, tokens), box (64, box_heads, box_tokens).
bool encode_map(EncodeTiledFn fn, CUtensorMap* map, bool bf16, const void* base, int headdim, int heads, int tokens,
                long long s_tok, long long s_head, int box_heads, int box_tokens) {
  cuuint64_t dims[3] = {(cuuint64_t)headdim, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)s_head * 2ull, (cuuint64_t)s_tok * 2ull};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int pick_nt(int kbs) {
  if (kbs <= 128) return kbs;
  for (int nt = 128; nt >= 16; nt -= 16)
    if (kbs % nt == 0) return nt;
  return 16;
}

}  // namespace

const char* sm100_ineligible_reason(const hbsa_forward_args& a, float scale) {
  if (a.dtype != HBSA_DTYPE_BF16 && a.dtype != HBSA_DTYPE_F16) return "dtype is not bf16/fp16";
  if (a.headdim != 64 && a.headdim != 128) return "headdim is not 64 or 128";
  if (!(scale > 0.f) || !isfinite(scale)) return "softmax_scale is not a positive finite number";
  if (a.q_stride[2] != 1 || a.k_stride[2] != 1 || a.v_stride[2] != 1 || a.o_stride[2] != 1)
    return "headdim stride is not 1";
  const int64_t strides[8] = {a.q_stride[0], a.q_stride[1], a.k_stride[0], a.k_stride[1],
                              a.v_stride[0], a.v_stride[1], a.o_stride[0], a.o_stride[1]};
  for (int i = 0; i < 8; ++i)
    if (strides[i] <= 0 || (strides[i] * 2) % 16 != 0) return "a token/head stride is not a positive multiple of 16 bytes";
  const uintptr_t ptrs[4] = {(uintptr_t)a.q, (uintptr_t)a.k, (uintptr_t)a.v, (uintptr_t)a.o};
  for (int i = 0; i < 4; ++i)
    if (ptrs[i] % 16 != 0) return "a tensor base address is not 16-byte aligned";
  return nullptr;
}

int launch_forward_sm100(const Problem& p, const Workspace& ws, const hbsa_forward_args& a, cudaStream_t stream,
                         const char** err_text) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { *err_text = "cuTensorMapEncodeTiled is not available from the CUDA driver"; return HBSA_ERR_DRIVER; }
  const bool bf16 = a.dtype == HBSA_DTYPE_BF16;

  Sm100Params P;
  P.p = p;
  P.ws = ws;
  P.o = a.o;
  P.o_s0 = a.o_stride[0];
  P.o_s1 = a.o_stride[1];
  P.nt = pick_nt(p.kbs);
  P.n_sub = p.kbs / P.nt;
  int gp = 1;
  while (gp < 128 && p.group % (gp * 2) == 0) gp *= 2;
  P.gp = gp;
  P.gp_shift = 0;
  while ((1 << P.gp_shift) < gp) ++P.gp_shift;
  P.n_head_sub = p.group / gp;
  P.tt = 128 / gp;
  P.tiles_per_qblock = (p.qbs + P.tt - 1) / P.tt;
  P.items_per_row = P.n_head_sub * P.tiles_per_qblock;
  P.scale_log2 = p.scale * 1.4426950408889634f;
  P.wait_budget = 4000000000ll;

  const long long items = (long long)p.nhead_k * p.num_q_block * P.items_per_row;
  if (items <= 0 || items > 0x7fffffffll) { *err_text = "too many work items for one launch"; return HBSA_ERR_SHAPE; }

  CUtensorMap tq, tk, tv;
  if (!encode_map(fn, &tq, bf16, a.q, p.headdim, p.nhead_q, a.total_q, a.q_stride[0], a.q_stride[1], gp, P.tt) ||
      !encode_map(fn, &tk, bf16, a.k, p.headdim, p.nhead_k, a.total_k, a.k_stride[0], a.k_stride[1], 1, P.nt) ||
      !encode_map(fn, &tv, bf16, a.v, p.headdim, p.nhead_k, a.total_k, a.v_stride[0], a.v_stride[1], 1, P.nt)) {
    *err_text = "cuTensorMapEncodeTiled rejected a q/k/v layout";
    return HBSA_ERR_UNSUPPORTED;
  }

  const size_t smem = 3u * 128u * (size_t)p.headdim * 2u + sizeof(Control) + 1024u;
  cudaError_t e = cudaSuccess;
#define HBSA_LAUNCH_SM100(D_, BF_)                                                                        \
  do {                                                                                                   \
    e = cudaFuncSetAttribute(fwd_sm100_kernel<D_, BF_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) {                                                                              \
      fwd_sm100_kernel<D_, BF_><<<(unsigned)items, kThreads, smem, stream>>>(tq, tk, tv, P);             \
      e = cudaGetLastError();                                                                            \
    }                                                                                                    \
  } while (0)
  if (p.headdim == 128) { if (bf16) HBSA_LAUNCH_SM100(128, true); else HBSA_LAUNCH_SM100(128, false); }
  else { if (bf16) HBSA_LAUNCH_SM100(64, true); else HBSA_LAUNCH_SM100(64, false); }
#undef HBSA_LAUNCH_SM100
  if (e != cudaSuccess) { *err_text = cudaGetErrorString(e); return (int)e; }
  return 0;
}

}  // namespace hbsa
