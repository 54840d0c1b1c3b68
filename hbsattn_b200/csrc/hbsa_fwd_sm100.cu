// Block-sparse attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces the two Triton kernels of the reference (fwd_triton_fix_tile_size.py:30-212,
// fwd_triton_auto_tile_size.py:76-251).  Differences of design, not of result:
//
//  * A work item is one 128-row M tile of one (kv-head, q-block): `TT = 128 / GP` tokens times
//    `GP` q-heads of the GQA group packed into the MMA M dimension, so that one K/V tile fetch
//    serves GP heads (the reference runs one program per q-head and re-reads K/V per head).
//  * One persistent CTA per SM pulls work items from an atomic cursor over the ItemRecord table the
//    schedule kernels wrote; the producer warp publishes each item to the other warps through a
//    two-slot ring in shared memory and runs up to one item ahead (Q is double-buffered).
//  * Only mask-active k-blocks are touched: the producer warp compacts the mask row with warp
//    ballots and issues TMA loads of exactly those K/V tiles into two-stage K and V rings (the
//    reference loops over all k-blocks of the sample and polls the mask byte,
//    fwd_triton_fix_tile_size.py:117-124).
//  * S = Q K^T and O += P V are tcgen05.mma instructions with fp32 accumulators in TMEM.  S is
//    double-buffered, so S(t+1) is computed while the softmax warps work on S(t); P (in the input
//    dtype, as at fwd_triton_fix_tile_size.py:187) is written back into TMEM over the S columns it
//    came from and consumed as the A operand of the second MMA, so it never touches shared memory.
//    O is double-buffered across items so that the epilogue of one item overlaps the next.
//  * Online softmax runs in registers on 256 threads: two threads per row, each owning half of the
//    tile's columns (row maxima are exchanged through shared memory), exp2 with the scale folded
//    in; the running output is rescaled only when a row maximum grows by more than 2^8.
//
// Warp roles (320 threads): warps 0-3 softmax columns [0, ca), warps 4-7 softmax columns [ca, nt)
// (TMEM lane quarter = warp id % 4), warp 8 work fetch + TMA producer, warp 9 TMEM allocator +
// MMA issuer.
//
// mbarriers.  T counts K/V tiles over the whole life of the CTA, I counts published items, Iq those
// of them that have tiles.  Two-entry barrier arrays are indexed by the low bit of the count and
// complete once per use, so a waiter for count c uses entry c & 1 and parity (c >> 1) & 1:
//   k_full / v_full [T]: TMA bytes landed          s_full [T]: S = Q K^T done (K stage free again)
//   p_full [T]: P written (one arrival per warp)   pv_done [T]: O += P V done (V stage, S buffer free)
//   q_full [Iq]: Q tile landed                     o_free [Iq]: epilogue has read O out of TMEM
//   item_full [I]: item slot written               item_done [I]: all consumers left item I
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>
#include <stdlib.h>
#include <type_traits>

#include "hbsa_common.cuh"
#include "sm100_ptx.cuh"

namespace hbsa {

namespace {

constexpr int kThreads = 320;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kTmemCols = 512;       // S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512)
constexpr int kTmemOCol = 256;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct Sm100Params {
  Problem p;
  Workspace ws;
  void* o;
  long long o_s0, o_s1;        // elements
  int nt;                      // rows of one K/V tile (multiple of 16, <= 128)
  int ca;                      // columns [0, ca) of a tile belong to softmax warps 0-3, [ca, nt) to warps 4-7
  int n_sub;                   // K/V tiles per k-block
  int gp, gp_shift;            // q-heads packed into one M tile
  int n_head_sub;              // group / gp
  int tt;                      // tokens per M tile = 128 / gp
  int tiles_per_qblock;
  int items_per_row;           // n_head_sub * tiles_per_qblock
  long long total_items;       // rows * items_per_row
  float scale_log2;
  long long wait_budget;       // clock64 ticks
  long long* trace;            // debugging aid: clock64 stamps of CTA 0 (NULL in normal use)
  int debug;                   // experiments (wrong results!): 1 = softmax does no math, 2 = K/V loaded only for the first tiles
};

constexpr int kTraceTiles = 96;      // tiles of CTA 0 that are stamped
constexpr int kTraceSlots = 32;      // stamps per tile (16..23: after every S MMA, 24..31: after every PV MMA)
// slot meanings: 0 K issued, 1 V issued, 2 MMA warp has K and a free S, 3 QK issued, 4 MMA warp has V and P,
// 5 PV issued, 6 softmax sees S, 7 row max done, 8 P written, 9 P arrival done, 10 item start (softmax), 11 epilogue done
__device__ __forceinline__ void stamp(long long* trace, int tile, int slot) {
  if (trace != nullptr && blockIdx.x == 0 && tile >= 0 && tile < kTraceTiles) trace[tile * kTraceSlots + slot] = clock64();
}

// What the producer tells the other warps about one work item.
struct ItemSlot {
  int n_tiles;        // < 0: no more work
  int tile_tok0;      // first token of the M tile (global)
  int head0;          // first q-head of the M tile
  int q_end;          // one past the last token of the q-block (global)
  int qi0;            // in-sample index of the tile's first token
  int k_len;
  int off;            // k_len - q_len
  int pad;
};

struct __align__(16) Control {
  unsigned long long item_full[2], item_done[2];
  unsigned long long q_full[2], k_full[2], v_full[2], s_full[2], p_full[2], pv_done[2], o_free[2];
  uint32_t tmem_base;
  int abort_flag;
  int tile_k0[4];
  ItemSlot slot[2];
  // Exchange between the two warps that share a TMEM lane quarter (the two threads of a row): values
  // go through these arrays, hand-over through the pair barriers (count 2, one arrival per warp) -
  // no thread ever spins on shared memory, which would steal bandwidth from the MMA operand reads.
  unsigned long long pair_max[2][4], pair_sum[2][4];   // [tile / item parity][quarter]
  float xmax[2][2][128];                // [tile parity][column half][row]: row maximum of tile T
  float xsum[2][2][128];                // [item parity][column half][row]: row sum of item Iq
};

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// P = exp2(S * scale - m) for `N` consecutive columns whose first tile column is c0; columns above
// col_limit are forced to zero.  Packs pairs to 16 bit and adds to four independent partial sums.
template <bool BF16, int N>
__device__ __forceinline__ void softmax_chunk(const uint32_t* r, uint32_t* pk, float scale_log2, float neg_m,
                                              int c0, int col_limit, float (&sum)[4]) {
  const bool full = col_limit >= c0 + N - 1;
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    float p0 = ptx::ex2_approx(fmaf(__uint_as_float(r[i]), scale_log2, neg_m));
    float p1 = ptx::ex2_approx(fmaf(__uint_as_float(r[i + 1]), scale_log2, neg_m));
    if (!full) {
      if (c0 + i > col_limit) p0 = 0.f;
      if (c0 + i + 1 > col_limit) p1 = 0.f;
    }
    sum[(i >> 1) & 1] += p0;
    sum[2 + ((i >> 1) & 1)] += p1;
    pk[i >> 1] = pack2<BF16>(p0, p1);
  }
}

// Row maximum over `N` columns into four independent partial maxima.
template <int N>
__device__ __forceinline__ void max_chunk(const uint32_t* r, int c0, int col_limit, float (&mx)[4]) {
  if (col_limit >= c0 + N - 1) {
#pragma unroll
    for (int i = 0; i < N; i += 8) {
      mx[0] = fmaxf(mx[0], fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
      mx[1] = fmaxf(mx[1], fmaxf(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])));
      mx[2] = fmaxf(mx[2], fmaxf(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])));
      mx[3] = fmaxf(mx[3], fmaxf(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      mx[i & 3] = fmaxf(mx[i & 3], (c0 + i <= col_limit) ? __uint_as_float(r[i]) : -INFINITY);
  }
}

// One lane polls the mbarrier, the rest of the warp sleeps at the shuffle instead of spinning.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, long long budget) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = ptx::mbar_wait_bounded(bar, parity, abort_flag, budget) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// Barrier entry and parity for the c-th use of a two-entry barrier array.
__device__ __forceinline__ uint32_t bar_of(uint32_t base, int c) { return base + 8u * (uint32_t)(c & 1); }
__device__ __forceinline__ uint32_t par_of(int c) { return (uint32_t)(c >> 1) & 1u; }

// The issue sequences of the MMA thread.  Every descriptor and TMEM address is precomputed into
// registers once per CTA, so a product is nothing but back-to-back tcgen05.mma instructions: the lone
// issuing thread needs several clocks per ordinary instruction and would otherwise starve the pipe.
template <int KSTEPS>
__device__ __forceinline__ void issue_qk(uint32_t tS, const uint64_t (&qd)[8], const uint64_t (&kd)[8], uint32_t idesc,
                                         long long* trace, int T) {
  ptx::mma_ss_c<false>(tS, qd[0], kd[0], idesc);
  stamp(trace, T, 16);
#pragma unroll
  for (int ks = 1; ks < KSTEPS; ++ks) { ptx::mma_ss_c<true>(tS, qd[ks], kd[ks], idesc); stamp(trace, T, 16 + ks); }
}
template <int KSTEPS>
__device__ __forceinline__ void issue_pv_steps(uint32_t tO, const uint32_t (&pa)[8], const uint64_t (&vd)[8], uint32_t idesc, bool first,
                                               long long* trace, int T) {
  if (first) ptx::mma_ts_c<false>(tO, pa[0], vd[0], idesc);
  else ptx::mma_ts_c<true>(tO, pa[0], vd[0], idesc);
  stamp(trace, T, 24);
#pragma unroll
  for (int ks = 1; ks < KSTEPS; ++ks) { ptx::mma_ts_c<true>(tO, pa[ks], vd[ks], idesc); stamp(trace, T, 24 + ks); }
}
__device__ __forceinline__ void issue_pv(int ksteps, uint32_t tO, const uint32_t (&pa)[8], const uint64_t (&vd)[8], uint32_t idesc, bool first,
                                         long long* trace, int T) {
  switch (ksteps) {
    case 1: issue_pv_steps<1>(tO, pa, vd, idesc, first, trace, T); break;
    case 2: issue_pv_steps<2>(tO, pa, vd, idesc, first, trace, T); break;
    case 3: issue_pv_steps<3>(tO, pa, vd, idesc, first, trace, T); break;
    case 4: issue_pv_steps<4>(tO, pa, vd, idesc, first, trace, T); break;
    case 5: issue_pv_steps<5>(tO, pa, vd, idesc, first, trace, T); break;
    case 6: issue_pv_steps<6>(tO, pa, vd, idesc, first, trace, T); break;
    case 7: issue_pv_steps<7>(tO, pa, vd, idesc, first, trace, T); break;
    default: issue_pv_steps<8>(tO, pa, vd, idesc, first, trace, T); break;
  }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Sm100Params P) {
  using namespace ptx;
  constexpr int PANELS = D / 64;
  constexpr uint32_t Q_BYTES = 128u * D * 2u;
  constexpr uint32_t KV_BYTES_MAX = 128u * D * 2u;
  const Problem& p = P.p;

  if (P.ws.status[0] != HBSA_STATUS_OK) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  OutT* const o_base = static_cast<OutT*>(P.o);

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* const smem = smem_raw + pad;
  const uint32_t sQ = raw_addr + pad;                 // 2 buffers
  const uint32_t sK = sQ + 2 * Q_BYTES;               // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES_MAX;          // 2 stages
  Control* const ctl = reinterpret_cast<Control*>(smem + 2 * Q_BYTES + 4 * KV_BYTES_MAX);
  const uint32_t bar_item_full = smem_u32(&ctl->item_full[0]), bar_item_done = smem_u32(&ctl->item_done[0]);
  const uint32_t bar_q_full = smem_u32(&ctl->q_full[0]), bar_k_full = smem_u32(&ctl->k_full[0]);
  const uint32_t bar_v_full = smem_u32(&ctl->v_full[0]), bar_s_full = smem_u32(&ctl->s_full[0]);
  const uint32_t bar_p_full = smem_u32(&ctl->p_full[0]), bar_pv_done = smem_u32(&ctl->pv_done[0]);
  const uint32_t bar_o_free = smem_u32(&ctl->o_free[0]);
  volatile int* const abort_flag = &ctl->abort_flag;
  volatile int* const tile_k0 = ctl->tile_k0;
  volatile ItemSlot* const slots = ctl->slot;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_item_full + 8 * i, 1);
      mbar_init(bar_item_done + 8 * i, 9);      // 8 softmax warps + the MMA warp
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_k_full + 8 * i, 1);
      mbar_init(bar_v_full + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 8);
      mbar_init(bar_pv_done + 8 * i, 1);
      mbar_init(bar_o_free + 8 * i, 8);
      for (int qd = 0; qd < 4; ++qd) {
        mbar_init(smem_u32(&ctl->pair_max[i][qd]), 2);
        mbar_init(smem_u32(&ctl->pair_sum[i][qd]), 2);
      }
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
  }

  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const long long budget = P.wait_budget;
  const uint32_t kv_tile_bytes = (uint32_t)P.nt * D * 2u;
  const uint32_t kv_panel_bytes = (uint32_t)P.nt * 128u;

  if (warp == kProducerWarp) {
    // =============================== work fetch + TMA producer ===============================
    const ItemRecord* const records = reinterpret_cast<const ItemRecord*>(P.ws.items);
    unsigned long long* const cursor = reinterpret_cast<unsigned long long*>(P.ws.cursor);
    int I = 0, Iq = 0, T = 0;
    bool ok = true;
    // one fetch ahead: the atomic and the record load of the next item overlap the current item
    long long next_idx = 0;
    if (lane == 0) next_idx = (long long)atomicAdd(cursor, 1ull);
    next_idx = __shfl_sync(0xffffffffu, next_idx, 0);
    while (ok) {
      const long long idx = next_idx;
      const bool have = idx < P.total_items;
      ItemRecord rec = {};
      int rem = 0;
      if (have) {
        rec = records[idx / P.items_per_row];
        rem = (int)(idx % P.items_per_row);
        if (lane == 0) next_idx = (long long)atomicAdd(cursor, 1ull);
        next_idx = __shfl_sync(0xffffffffu, next_idx, 0);
      }
      const int hsub = rem / P.tiles_per_qblock, qt = rem % P.tiles_per_qblock;
      const int tile_tok0 = rec.q_begin + qt * P.tt;
      if (have && tile_tok0 >= rec.q_end) continue;          // M tile past the ragged end of the q-block
      const int head0 = rec.hk * p.group + hsub * P.gp;
      const int n_tiles = have ? rec.n_tiles : -1;

      // publish: slot I & 1 is free once every consumer has left item I - 2
      if (I >= 2) ok = warp_wait(bar_of(bar_item_done, I), par_of(I - 2), abort_flag, budget);
      if (!ok) break;
      if (lane == 0) {
        volatile ItemSlot* sl = &slots[I & 1];
        sl->n_tiles = n_tiles;
        sl->tile_tok0 = tile_tok0;
        sl->head0 = head0;
        sl->q_end = rec.q_end;
        sl->qi0 = rec.q_in0 + qt * P.tt;
        sl->k_len = rec.k_len;
        sl->off = rec.off;
        __threadfence_block();
        mbar_arrive(bar_of(bar_item_full, I));
      }
      ++I;
      if (!have) break;
      if (n_tiles <= 0) continue;

      // The first K tile of the item goes to stage T & 1, free once S(T-2) is done; the S products are
      // issued in order, so this also means that the item that last used Q buffer Iq & 1 is through
      // with it (its last tile is T-2 or earlier).
      if (T >= 2) ok = warp_wait(bar_of(bar_s_full, T), par_of(T - 2), abort_flag, budget);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(bar_of(bar_q_full, Iq), Q_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(sQ + (Iq & 1) * Q_BYTES + pn * (128u * 128u), &tm_q, bar_of(bar_q_full, Iq), pn * 64, head0, tile_tok0);
      }
      ++Iq;
      const uint8_t* mrow = p.mask + rec.hk * p.mask_s0 + rec.qb * p.mask_s1;
      bool bit_next = lane < rec.n_reach && mrow[(long long)(rec.kb0 + lane) * p.mask_s2] != 0;
      for (int base = 0; base < rec.n_reach && ok; base += 32) {
        uint32_t bal = __ballot_sync(0xffffffffu, bit_next);
        {                                                   // mask bytes of the next 32 k-blocks, one chunk ahead
          const int jn = base + 32 + lane;
          bit_next = jn < rec.n_reach && mrow[(long long)(rec.kb0 + jn) * p.mask_s2] != 0;
        }
        while (bal != 0 && ok) {
          const int jj = base + __ffs(bal) - 1;
          bal &= bal - 1;
          const int blk_k0 = jj * p.kbs;
          for (int sub = 0; sub < P.n_sub && ok; ++sub) {
            const int k0 = blk_k0 + sub * P.nt;
            if (k0 >= rec.k_len) break;
            if (T >= 2) ok = warp_wait(bar_of(bar_s_full, T), par_of(T - 2), abort_flag, budget);
            if (!ok) break;
            if (lane == 0) {
              tile_k0[T & 3] = k0;
              __threadfence_block();
              if ((P.debug & 2) && T >= 2) mbar_arrive(bar_of(bar_k_full, T));
              else mbar_arrive_expect_tx(bar_of(bar_k_full, T), kv_tile_bytes);
#pragma unroll
              for (int pn = 0; pn < PANELS; ++pn)
                if (!((P.debug & 2) && T >= 2)) tma_load_3d(sK + (T & 1) * KV_BYTES_MAX + pn * kv_panel_bytes, &tm_k, bar_of(bar_k_full, T), pn * 64, rec.hk, rec.k_begin + k0);
              stamp(P.trace, T, 0);
            }
            if (T >= 2) ok = warp_wait(bar_of(bar_pv_done, T), par_of(T - 2), abort_flag, budget);
            if (!ok) break;
            if (lane == 0) {
              if ((P.debug & 2) && T >= 2) mbar_arrive(bar_of(bar_v_full, T));
              else mbar_arrive_expect_tx(bar_of(bar_v_full, T), kv_tile_bytes);
#pragma unroll
              for (int pn = 0; pn < PANELS; ++pn)
                if (!((P.debug & 2) && T >= 2)) tma_load_3d(sV + (T & 1) * KV_BYTES_MAX + pn * kv_panel_bytes, &tm_v, bar_of(bar_v_full, T), pn * 64, rec.hk, rec.k_begin + k0);
              stamp(P.trace, T, 1);
            }
            ++T;
          }
        }
      }
    }
    if (!ok) {
      // Gave up: let the copies already issued land before the CTA retires (bounded).
      for (int back = 1; back <= 2 && T - back >= 0; ++back) {
        mbar_wait_bounded(bar_of(bar_k_full, T - back), par_of(T - back), abort_flag, budget >> 4);
        mbar_wait_bounded(bar_of(bar_v_full, T - back), par_of(T - back), abort_flag, budget >> 4);
      }
    }
  } else if (warp == kMmaWarp) {
    // =============================== MMA issuer ===============================
    // One thread runs an event loop: whichever of "the oldest P V product whose P is written" and "the
    // next S = Q K^T whose K tile has landed and whose S buffer is free" is ready gets issued, so the
    // tensor pipe works on S(t+1) while the softmax warps are busy with S(t) and P V(t) starts the
    // moment P(t) exists.  All probes are non-blocking; a clock budget bounds the loop.
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc(BF16, false, false, 128, P.nt);
      const uint32_t idesc_pv = make_idesc(BF16, false, true, 128, D);
      const int ksteps_pv = P.nt >> 4;
      const int ca_steps = P.ca >> 4;
      const uint32_t p_jump = (uint32_t)P.ca >> 1;                 // P of columns [ca, nt) starts at S + ca
      const uint32_t desc_hi = smem_desc_hi(1024u);
      const uint32_t kpanel_units = kv_panel_bytes >> 4;
      // Q and K are K-major: 16 head dims further = 32 bytes = 2 descriptor units inside a 64-dim panel.
      // V is MN-major: 16 keys further = 2048 bytes = 128 units.  P: 8 TMEM columns per 16 keys, columns
      // [0, ca) at S + 0.., columns [ca, nt) at S + ca..
      uint64_t qd0[8], qd1[8], kd0[8], kd1[8], vd0[8], vd1[8];
      uint32_t pa0[8], pa1[8];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t ko = (uint32_t)(ks >> 2) * kpanel_units + (uint32_t)(ks & 3) * 2u;
        const uint32_t qo = (uint32_t)(ks >> 2) * 1024u + (uint32_t)(ks & 3) * 2u;
        qd0[ks] = smem_desc_join(smem_desc_lo(sQ, 16u) + qo, desc_hi);
        qd1[ks] = smem_desc_join(smem_desc_lo(sQ + Q_BYTES, 16u) + qo, desc_hi);
        kd0[ks] = smem_desc_join(smem_desc_lo(sK, 16u) + ko, desc_hi);
        kd1[ks] = smem_desc_join(smem_desc_lo(sK + KV_BYTES_MAX, 16u) + ko, desc_hi);
        vd0[ks] = smem_desc_join(smem_desc_lo(sV, kv_panel_bytes) + (uint32_t)ks * 128u, desc_hi);
        vd1[ks] = smem_desc_join(smem_desc_lo(sV + KV_BYTES_MAX, kv_panel_bytes) + (uint32_t)ks * 128u, desc_hi);
        const uint32_t po = (uint32_t)ks * 8u + (ks >= ca_steps ? p_jump : 0u);
        pa0[ks] = tmem_base + po;
        pa1[ks] = tmem_base + 128u + po;
      }
      int I = 0, Iq = 0, T = 0;
      bool have_item = false, finished = false, first = false;
      int n_left = 0;
      // P V products that have their S issued but are not issued themselves (at most two: T-2 is done
      // before S(T) may start), oldest first
      int pv_T[2] = {-1, -1}, pv_first[2] = {0, 0}, pv_iq[2] = {0, 0}, pv_n = 0;
      long long t_progress = clock64();
      while (true) {
        bool progress = false;
        if (!have_item && !finished && mbar_test(bar_of(bar_item_full, I), par_of(I))) {
          const int n_tiles = slots[I & 1].n_tiles;
          if (n_tiles < 0) {
            finished = true;
          } else if (n_tiles == 0) {
            mbar_arrive(bar_of(bar_item_done, I));
            ++I;
          } else {
            have_item = true;
            first = true;
            n_left = n_tiles;
          }
          progress = true;
        }
        if (pv_n > 0) {
          const int pT = pv_T[0];
          bool ready = mbar_test(bar_of(bar_p_full, pT), par_of(pT)) && mbar_test(bar_of(bar_v_full, pT), par_of(pT));
          // the first P V of an item overwrites O: the epilogue of the item two before must have read it
          if (ready && pv_first[0] && pv_iq[0] >= 2) ready = mbar_test(bar_of(bar_o_free, pv_iq[0]), par_of(pv_iq[0] - 2));
          if (ready) {
            tc_fence_after();
            stamp(P.trace, pT, 4);
            const uint32_t tOb = tmem_base + kTmemOCol + (uint32_t)(pv_iq[0] & 1) * 128u;
            if (pT & 1) issue_pv(ksteps_pv, tOb, pa1, vd1, idesc_pv, pv_first[0] != 0, P.trace, pT);
            else issue_pv(ksteps_pv, tOb, pa0, vd0, idesc_pv, pv_first[0] != 0, P.trace, pT);
            tc_commit(bar_of(bar_pv_done, pT));
            stamp(P.trace, pT, 5);
            pv_T[0] = pv_T[1]; pv_first[0] = pv_first[1]; pv_iq[0] = pv_iq[1];
            --pv_n;
            progress = true;
          }
        }
        if (have_item && pv_n < 2) {
          bool ready = mbar_test(bar_of(bar_k_full, T), par_of(T));
          if (ready && first) ready = mbar_test(bar_of(bar_q_full, Iq), par_of(Iq));
          // S buffer T & 1 held P(T-2): free once PV(T-2) is done
          if (ready && T >= 2) ready = mbar_test(bar_of(bar_pv_done, T), par_of(T - 2));
          if (ready) {
            tc_fence_after();
            stamp(P.trace, T, 2);
            const uint32_t tSb = tmem_base + (uint32_t)(T & 1) * 128u;
            if (Iq & 1) {
              if (T & 1) issue_qk<D / 16>(tSb, qd1, kd1, idesc_qk, P.trace, T);
              else issue_qk<D / 16>(tSb, qd1, kd0, idesc_qk, P.trace, T);
            } else {
              if (T & 1) issue_qk<D / 16>(tSb, qd0, kd1, idesc_qk, P.trace, T);
              else issue_qk<D / 16>(tSb, qd0, kd0, idesc_qk, P.trace, T);
            }
            tc_commit(bar_of(bar_s_full, T));
            stamp(P.trace, T, 3);
            pv_T[pv_n] = T; pv_first[pv_n] = first ? 1 : 0; pv_iq[pv_n] = Iq;
            ++pv_n;
            ++T;
            first = false;
            if (--n_left == 0) {
              mbar_arrive(bar_of(bar_item_done, I));
              ++I;
              ++Iq;
              have_item = false;
            }
            progress = true;
          }
        }
        if (finished && pv_n == 0) break;
        if (progress) {
          t_progress = clock64();
        } else {
          if (*abort_flag) break;
          if (clock64() - t_progress > budget) { *abort_flag = 1; break; }
        }
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax + epilogue ===============================
    const int half = tid >> 7;                       // 0: columns [0, ca), 1: columns [ca, nt)
    const int row = tid & 127;
    const int quarter = warp & 3;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int my_c0 = half == 0 ? 0 : P.ca;          // first tile column of this thread
    const int my_nc = half == 0 ? P.ca : P.nt - P.ca; // columns of this thread: 0, 16, 32, 48 or 64
    const float scale_log2 = P.scale_log2;
    int I = 0, Iq = 0, T = 0;
    bool ok = true;
    while (ok) {
      ok = warp_wait(bar_of(bar_item_full, I), par_of(I), abort_flag, budget);
      if (!ok) break;
      const int n_tiles = slots[I & 1].n_tiles;
      if (n_tiles < 0) break;
      const int r_tok = slots[I & 1].tile_tok0 + (row >> P.gp_shift);
      const int r_head = slots[I & 1].head0 + (row & (P.gp - 1));
      const bool r_valid = r_tok < slots[I & 1].q_end;
      // each of the two threads of a row stores half of the head dimension
      OutT* const orow = o_base + r_tok * P.o_s0 + r_head * P.o_s1 + half * (D / 2);
      if (n_tiles == 0) {
        // No active k-block: the rows are exact zeros (fwd_triton_fix_tile_size.py:189).
        if (r_valid) {
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int i = 0; i < D / 16; ++i) dst[i] = make_uint4(0, 0, 0, 0);
        }
      } else {
        const uint32_t tO = tmem_base + kTmemOCol + (uint32_t)(Iq & 1) * 128u + lane_off;
        int limit_row = slots[I & 1].k_len - 1;
        if (p.causal) limit_row = min(limit_row, slots[I & 1].qi0 + (row >> P.gp_shift) + slots[I & 1].off);
        float m_ref = -INFINITY, l = 0.f;
        if (tid == 0) stamp(P.trace, T, 10);
        for (int t = 0; t < n_tiles && ok; ++t, ++T) {
          ok = warp_wait(bar_of(bar_s_full, T), par_of(T), abort_flag, budget);
          if (!ok) break;
          tc_fence_after();
          if (tid == 0) stamp(P.trace, T, 6);
          const int col_limit = limit_row - tile_k0[T & 3];            // tile columns <= col_limit are valid
          const uint32_t tSmine = tmem_base + (uint32_t)(T & 1) * 128u + lane_off + (uint32_t)my_c0;

          // ---- this thread's columns of S, all in registers
          uint32_t r[64];
          if (my_nc >= 32) tmem_ld32(tSmine, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          if (my_nc >= 64) tmem_ld32(tSmine + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          if (my_nc == 16) tmem_ld16(tSmine, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
          if (my_nc == 48) tmem_ld16(tSmine + 32, *reinterpret_cast<uint32_t(*)[16]>(&r[32]));
          tmem_wait_ld();
          if (tid == 0) stamp(P.trace, T, 12);
          if (P.debug & 1) {
            if (my_nc >= 32) tmem_st16(tSmine, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
            if (my_nc >= 64) tmem_st16(tSmine + 16, *reinterpret_cast<uint32_t(*)[16]>(&r[32]));
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_of(bar_p_full, T));
            if (tid == 0) stamp(P.trace, T, 9);
            continue;
          }

          // ---- row maximum: own columns, then the other half's through shared memory
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (my_nc >= 32) max_chunk<32>(&r[0], my_c0, col_limit, mx4);
          if (my_nc >= 64) max_chunk<32>(&r[32], my_c0 + 32, col_limit, mx4);
          if (my_nc == 16) max_chunk<16>(&r[0], my_c0, col_limit, mx4);
          if (my_nc == 48) max_chunk<16>(&r[32], my_c0 + 32, col_limit, mx4);
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          if (tid == 0) stamp(P.trace, T, 13);
          {
            ctl->xmax[T & 1][half][row] = mx;
            __syncwarp();
            const uint32_t pb = smem_u32(&ctl->pair_max[T & 1][quarter]);
            if (lane == 0) mbar_arrive(pb);
            ok = warp_wait(pb, par_of(T), abort_flag, budget);
            if (!ok) break;
            mx = fmaxf(mx, *reinterpret_cast<volatile float*>(&ctl->xmax[T & 1][half ^ 1][row]));
          }
          if (tid == 0) stamp(P.trace, T, 7);
          const float mx_s = mx * scale_log2;                          // scale > 0 keeps the order
          if (t == 0) {
            m_ref = mx_s;
          } else {
            const bool need = mx_s > m_ref + kRescaleThreshold;
            if (__any_sync(0xffffffffu, need)) {
              // O and l move to the new reference maximum; needs O += P V of the previous tile.
              // Both warps of a row pair take this branch together (same maxima) and split O's columns.
              ok = warp_wait(bar_of(bar_pv_done, T - 1), par_of(T - 1), abort_flag, budget);
              if (!ok) break;
              tc_fence_after();
              const float alpha = need ? ex2_approx(m_ref - mx_s) : 1.f;
#pragma unroll
              for (int c0 = 0; c0 < D / 2; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tO + half * (D / 2) + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st32(tO + half * (D / 2) + c0, o);
              }
              tmem_wait_st();
              l *= alpha;
              if (need) m_ref = mx_s;
            }
          }
          const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;

          // ---- P = exp2(S * scale - m) packed to 16 bit over this thread's own S columns, row sum
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          uint32_t pk[32];
          if (my_nc >= 32) {
            softmax_chunk<BF16, 32>(&r[0], &pk[0], scale_log2, neg_m, my_c0, col_limit, sum);
            tmem_st16(tSmine, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
          }
          if (my_nc >= 64) {
            softmax_chunk<BF16, 32>(&r[32], &pk[16], scale_log2, neg_m, my_c0 + 32, col_limit, sum);
            tmem_st16(tSmine + 16, *reinterpret_cast<uint32_t(*)[16]>(&pk[16]));
          }
          if (my_nc == 16) {
            softmax_chunk<BF16, 16>(&r[0], &pk[0], scale_log2, neg_m, my_c0, col_limit, sum);
            tmem_st8(tSmine, *reinterpret_cast<uint32_t(*)[8]>(&pk[0]));
          }
          if (my_nc == 48) {
            softmax_chunk<BF16, 16>(&r[32], &pk[16], scale_log2, neg_m, my_c0 + 32, col_limit, sum);
            tmem_st8(tSmine + 16, *reinterpret_cast<uint32_t(*)[8]>(&pk[16]));
          }
          l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
          tmem_wait_st();
          tc_fence_before();
          if (tid == 0) stamp(P.trace, T, 8);
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_of(bar_p_full, T));             // one arrival per warp
          if (tid == 0) stamp(P.trace, T, 9);
        }
        if (!ok) break;

        // ---- epilogue: the row sum is the sum of both halves; O / l -> global with 16-byte stores,
        //      rows past the q-block end are dropped
        {
          ctl->xsum[Iq & 1][half][row] = l;
          __syncwarp();
          const uint32_t pb = smem_u32(&ctl->pair_sum[Iq & 1][quarter]);
          if (lane == 0) mbar_arrive(pb);
          ok = warp_wait(pb, par_of(Iq), abort_flag, budget);
          if (!ok) break;
          l += *reinterpret_cast<volatile float*>(&ctl->xsum[Iq & 1][half ^ 1][row]);
        }
        ok = warp_wait(bar_of(bar_pv_done, T - 1), par_of(T - 1), abort_flag, budget);
        if (!ok) break;
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        uint32_t oa[32], ob[32];
        tmem_ld32(tO + half * (D / 2), oa);
        if (D == 128) tmem_ld32(tO + half * (D / 2) + 32, ob);
        tmem_wait_ld();
        tc_fence_before();                                               // O is in registers: the buffer may be overwritten
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_of(bar_o_free, Iq));
        if (r_valid) {
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            const uint32_t* rr = i < 4 ? oa : ob;
            const int b = (i & 3) * 8;
            uint32_t w0 = pack2<BF16>(__uint_as_float(rr[b]) * inv, __uint_as_float(rr[b + 1]) * inv);
            uint32_t w1 = pack2<BF16>(__uint_as_float(rr[b + 2]) * inv, __uint_as_float(rr[b + 3]) * inv);
            uint32_t w2 = pack2<BF16>(__uint_as_float(rr[b + 4]) * inv, __uint_as_float(rr[b + 5]) * inv);
            uint32_t w3 = pack2<BF16>(__uint_as_float(rr[b + 6]) * inv, __uint_as_float(rr[b + 7]) * inv);
            if (!(l > 0.f)) w0 = w1 = w2 = w3 = 0u;      // rows that saw no key are exact zeros
            dst[i] = make_uint4(w0, w1, w2, w3);
          }
        }
        ++Iq;
      }
      if (tid == 0) stamp(P.trace, T - 1, 11);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_of(bar_item_done, I));
      ++I;
    }
  }

  // ---- teardown: every thread gets here (all waits are bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
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

long long* g_trace = nullptr;

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace

void sm100_set_trace(long long* device_buffer) { g_trace = device_buffer; }
size_t sm100_trace_bytes() { return (size_t)kTraceTiles * kTraceSlots * sizeof(long long); }

int sm100_kv_tile_rows(int kbs) {
  if (kbs <= 128) return kbs;
  for (int nt = 128; nt >= 16; nt -= 16)
    if (kbs % nt == 0) return nt;
  return 16;
}

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
  P.nt = sm100_kv_tile_rows(p.kbs);
  P.ca = ((P.nt / 16 + 1) / 2) * 16;                           // first half of the 16-column groups, rounded up
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
  P.trace = g_trace;
  { const char* dbg = getenv("HBSA_DEBUG"); P.debug = dbg ? atoi(dbg) : 0; }

  P.total_items = (long long)p.nhead_k * p.num_q_block * P.items_per_row;
  if (P.total_items <= 0) { *err_text = "no work items"; return HBSA_ERR_SHAPE; }
  const long long resident = sm_count();                        // one persistent CTA per SM
  const unsigned grid = (unsigned)(P.total_items < resident ? P.total_items : resident);

  CUtensorMap tq, tk, tv;
  if (!encode_map(fn, &tq, bf16, a.q, p.headdim, p.nhead_q, a.total_q, a.q_stride[0], a.q_stride[1], gp, P.tt) ||
      !encode_map(fn, &tk, bf16, a.k, p.headdim, p.nhead_k, a.total_k, a.k_stride[0], a.k_stride[1], 1, P.nt) ||
      !encode_map(fn, &tv, bf16, a.v, p.headdim, p.nhead_k, a.total_k, a.v_stride[0], a.v_stride[1], 1, P.nt)) {
    *err_text = "cuTensorMapEncodeTiled rejected a q/k/v layout";
    return HBSA_ERR_UNSUPPORTED;
  }

  const size_t smem = 6u * 128u * (size_t)p.headdim * 2u + sizeof(Control) + 1024u;
  cudaError_t e = cudaSuccess;
#define HBSA_LAUNCH_SM100(D_, BF_)                                                                        \
  do {                                                                                                   \
    e = cudaFuncSetAttribute(fwd_sm100_kernel<D_, BF_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) {                                                                              \
      fwd_sm100_kernel<D_, BF_><<<grid, kThreads, smem, stream>>>(tq, tk, tv, P);                         \
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
