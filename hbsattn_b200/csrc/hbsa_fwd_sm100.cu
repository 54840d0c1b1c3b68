// Block-sparse attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces the two Triton kernels of the reference (fwd_triton_fix_tile_size.py:30-212,
// fwd_triton_auto_tile_size.py:76-251).  Differences of design, not of result:
//
//  * A work item is one 128-row M tile of one (kv-head, q-block): `TT = 128 / GP` tokens times
//    `GP` q-heads of the GQA group packed into the MMA M dimension, so that one K/V tile fetch
//    serves GP heads (the reference runs one program per q-head and re-reads K/V per head).
//  * Persistent CTAs, two per SM, pull work items from an atomic cursor over the ItemRecord table the
//    schedule kernels wrote; the producer warp publishes each item to the other warps through a
//    two-slot ring in shared memory and runs ahead of them.  Two CTAs per SM mean two independent
//    items in flight, so the start and the end of one item hide behind the tiles of the other.
//  * Only mask-active k-blocks are touched: the producer warp compacts the mask row with warp
//    ballots and issues TMA loads of exactly those K/V tiles (at most 64 rows each) into two-stage K
//    and V rings (the reference loops over all k-blocks of the sample and polls the mask byte,
//    fwd_triton_fix_tile_size.py:117-124).
//  * S = Q K^T and O += P V are tcgen05.mma instructions with fp32 accumulators in TMEM.  S is
//    double-buffered, so S(t+1) is computed while the softmax warps work on S(t); P (in the input
//    dtype, as at fwd_triton_fix_tile_size.py:187) is written back into TMEM over the S columns it
//    came from and consumed as the A operand of the second MMA, so it never touches shared memory.
//    One thread issues every MMA; because tcgen05.mma instructions of one thread execute in issue
//    order, S(t+2) is issued right behind P V(t) into the buffer that P(t) occupies without waiting
//    for P V(t) to complete (HBSA_STRICT_TCGEN05 builds wait and fence instead; they exist to check this
//    ordering bit for bit).  The issuing thread blocks until the tensor pipe's queue takes an instruction, so the
//    twelve instructions of a 64-row tile occupy it for as long as the products of both resident CTAs occupy the
//    pipe (measured: about half of the tile period); it looks for new inputs between the two products only,
//    and its polling loop is kept to one probe per turn.
//  * Online softmax in registers, one thread per row: tcgen05.ld of the tile's <= 64 columns, in-place
//    -inf masking on diagonal / ragged tiles, exp2 with the scale folded in, fp32 row sum; no shuffles
//    and no shared-memory exchange.  The exponentials of a tile run against the reference maximum of the
//    previous tiles; only when the tile's row sum (which bounds every P of the row) exceeds 2^14 is the row
//    maximum computed, and the running output rescaled in TMEM (and the tile redone) where it grew by more
//    than 2^8.  The arithmetic around the exponentials is two-wide (fma/add/mul.rn.f32x2).
//  * The last CTA to leave rewinds the work cursor, so one schedule serves any number of launches.  With
//    `lse` set, ln sum exp of every row goes out beside O.
//
// Warp roles (192 threads): warps 0-3 softmax + epilogue (TMEM lane quarter = warp id), warp 4 work
// fetch + TMA producer, warp 5 TMEM allocator + MMA issuer.  TMEM (256 columns): S0 [0,64), S1 [64,128),
// O [128,256).  The kernel is instantiated for tiles of 64, 128 and 256 head dimensions; other head dimensions
// (multiples of 8) run on the next larger one with the surplus columns zero-filled by the TMA boxes.  At 256 a CTA
// takes 512 TMEM columns (O [128,384)) and 192 KB of shared memory, i.e. one CTA per SM.
//
// mbarriers.  T counts K/V tiles over the whole life of the CTA, I counts published items, Iq those
// of them that have tiles.  Two-entry barrier arrays are indexed by the low bit of the count and
// complete once per use, so a waiter for count c uses entry c & 1 and parity (c >> 1) & 1:
//   k_full / v_full [T]: TMA bytes landed          s_full [T]: S = Q K^T done (K stage free again)
//   pv_done [T]: O += P V done (V stage free again)
// P(T) is handed over through a plain shared-memory counter instead (p_count, one increment per softmax warp, never
// reset): the issuing thread reads it with an ordinary load in its polling loop.
//   q_full [Iq]: Q tile landed                     o_free [Iq]: epilogue has read O out of TMEM
//   item_full [I]: item slot written               item_done [I]: all consumers left item I
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>
#include <stdlib.h>
#include <mutex>
#include <type_traits>

#include "hbsa_common.cuh"
#include "sm100_ptx.cuh"

namespace hbsa {

namespace {

constexpr int kThreads = 192;
constexpr int kSoftmaxWarps = 4;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kTileRowsMax = 64;      // rows of a K/V tile
// S0, S1 of 64 columns + O of D columns, rounded up to a power of two
template <int D> struct TmemCols { static constexpr uint32_t value = D > 128 ? 512u : 256u; };
constexpr uint32_t kSStride = 64u;    // TMEM columns between the two S buffers
constexpr uint32_t kTmemOCol = 128u;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct Sm100Params {
  Problem p;
  Workspace ws;
  void* o;
  long long o_s0, o_s1;        // elements
  float* lse;                  // NULL or [total_q, nhead_q]: natural-log sum of exponentials per row
  int total_q;
  int nt;                      // rows of one K/V tile (multiple of 16, <= 64)
  int n_sub;                   // K/V tiles per k-block
  int gp, gp_shift;            // q-heads packed into one M tile
  int n_head_sub;              // group / gp
  int tt;                      // tokens per M tile = 128 / gp
  int tiles_per_qblock;
  int o_vec32;                 // output rows are 32-byte aligned: 256-bit stores
  int items_per_row;           // n_head_sub * tiles_per_qblock
  long long total_items;       // rows * items_per_row
  float scale_log2;
  long long wait_budget;       // clock64 ticks
  int debug_stall;             // debugging aid: the producer publishes nothing, every wait runs out
  long long* trace;            // debugging aid: clock64 stamps of CTA 0 (NULL in normal use)
};

constexpr int kTraceTiles = 96;      // tiles of CTA 0 that are stamped
constexpr int kTraceSlots = 32;      // stamps per tile
constexpr int kTraceCtas = 512;      // behind the tile stamps: start time (ns) and SM of the first CTAs
// slots: 0 K issued, 1 V issued, 2 S(t) issue starts, 3 S(t) issued, 4 PV(t) issue starts, 5 PV(t) issued,
// 6 softmax sees S, 7 row max done, 8 P written, 9 P arrival done, 10 item start, 11 epilogue done,
// 12 S in registers, 13 epilogue starts, 17 issuer sees P, 18 issuer sees V, 22 last PV seen complete, 23 O in registers
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
  unsigned long long q_full[2], k_full[2], v_full[2], s_full[2], pv_done[2], o_free[2];
  unsigned long long drain;
  uint32_t tmem_base;
  int abort_flag;
  unsigned p_count[2];       // arrivals of the softmax warps for the S buffer tile & 1 (never reset: 4 per tile)
  int tile_k0[4];
  ItemSlot slot[2];
};

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// The softmax of one thread works on 16-column groups of its row (one TMEM load / store each), so that
// a single copy of the code serves every tile width; masked columns are set to -inf beforehand, which
// exp2 turns into exact zeros.
__device__ __forceinline__ void max16(const uint32_t* r, float (&mx)[4]) {
  mx[0] = max3(mx[0], __uint_as_float(r[0]), __uint_as_float(r[1]));
  mx[1] = max3(mx[1], __uint_as_float(r[2]), __uint_as_float(r[3]));
  mx[2] = max3(mx[2], __uint_as_float(r[4]), __uint_as_float(r[5]));
  mx[3] = max3(mx[3], __uint_as_float(r[6]), __uint_as_float(r[7]));
  mx[0] = max3(mx[0], __uint_as_float(r[8]), __uint_as_float(r[9]));
  mx[1] = max3(mx[1], __uint_as_float(r[10]), __uint_as_float(r[11]));
  mx[2] = max3(mx[2], __uint_as_float(r[12]), __uint_as_float(r[13]));
  mx[3] = max3(mx[3], __uint_as_float(r[14]), __uint_as_float(r[15]));
}
// P = exp2(S * scale - m) for 16 columns, packed to 16-bit pairs; four independent partial row sums.
// The scale-and-shift and the sums use the two-wide fp32 instructions: same FMA-pipe time, half the issue
// slots.
template <bool BF16>
__device__ __forceinline__ void exp16(const uint32_t* r, uint32_t (&pk)[8], float scale_log2, float neg_m, float (&sum)[4]) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2), neg_m2 = ptx::pack_f32x2(neg_m, neg_m);
  uint64_t sa = ptx::pack_f32x2(sum[0], sum[2]), sb = ptx::pack_f32x2(sum[1], sum[3]);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    float x0, x1;
    ptx::unpack_f32x2(ptx::fma_f32x2(ptx::pack_b32x2(r[i], r[i + 1]), scale2, neg_m2), x0, x1);
    const float p0 = ptx::ex2_approx(x0), p1 = ptx::ex2_approx(x1);
    if ((i >> 1) & 1) sb = ptx::add_f32x2(sb, ptx::pack_f32x2(p0, p1));
    else sa = ptx::add_f32x2(sa, ptx::pack_f32x2(p0, p1));
    pk[i >> 1] = pack2<BF16>(p0, p1);
  }
  ptx::unpack_f32x2(sa, sum[0], sum[2]);
  ptx::unpack_f32x2(sb, sum[1], sum[3]);
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
// registers once per CTA, so a product is nothing but back-to-back tcgen05.mma instructions.
template <int KSTEPS>
__device__ __forceinline__ void issue_qk(uint32_t tS, const uint64_t (&qd)[KSTEPS], const uint64_t (&kd)[KSTEPS], uint32_t idesc) {
  ptx::mma_ss_c<false>(tS, qd[0], kd[0], idesc);
#pragma unroll
  for (int ks = 1; ks < KSTEPS; ++ks) ptx::mma_ss_c<true>(tS, qd[ks], kd[ks], idesc);
}
// N k-steps of O (+)= P V; the first one overwrites O when `first`.
template <int N>
__device__ __forceinline__ void issue_pv_n(uint32_t tO, const uint32_t (&pa)[4], const uint64_t (&vd)[4], uint32_t idesc, bool first) {
  if (first) ptx::mma_ts_c<false>(tO, pa[0], vd[0], idesc);
  else ptx::mma_ts_c<true>(tO, pa[0], vd[0], idesc);
#pragma unroll
  for (int ks = 1; ks < N; ++ks) ptx::mma_ts_c<true>(tO, pa[ks], vd[ks], idesc);
}
__device__ __forceinline__ void issue_pv(int n, uint32_t tO, const uint32_t (&pa)[4], const uint64_t (&vd)[4], uint32_t idesc, bool first) {
  switch (n) {
    case 1: issue_pv_n<1>(tO, pa, vd, idesc, first); break;
    case 2: issue_pv_n<2>(tO, pa, vd, idesc, first); break;
    case 3: issue_pv_n<3>(tO, pa, vd, idesc, first); break;
    default: issue_pv_n<4>(tO, pa, vd, idesc, first); break;
  }
}

// TRACE = true is the instantiation that runs while a debug trace buffer is set; the shipped path carries
// no stamp code at all.
// NT > 0 fixes the rows of a K/V tile at compile time (the common 64-row case then has no branches on the tile
// width); NT = 0 reads them from the parameters.
template <int D, bool BF16, bool TRACE, int NT>
__global__ void __launch_bounds__(kThreads, 2)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Sm100Params P) {
  using namespace ptx;
  constexpr int PANELS = D / 64;
  constexpr uint32_t Q_BYTES = 128u * D * 2u;
  constexpr uint32_t KV_BYTES_MAX = (uint32_t)kTileRowsMax * D * 2u;
  const Problem& p = P.p;
  using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  OutT* const o_base = static_cast<OutT*>(P.o);

  if (P.ws.status[0] != HBSA_STATUS_OK) {
    zero_fill_output(o_base, P.o_s0, P.o_s1, 1ll, P.total_q, p.nhead_q, p.headdim, P.lse);
    return;
  }
  if (TRACE && P.trace != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceCtas) {
    unsigned long long ns;
    uint32_t smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    P.trace[kTraceTiles * kTraceSlots + blockIdx.x] = (long long)ns;
    P.trace[kTraceTiles * kTraceSlots + kTraceCtas + blockIdx.x] = (long long)smid;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* const smem = smem_raw + pad;
  const uint32_t sQ = raw_addr + pad;
  const uint32_t sK = sQ + Q_BYTES;                   // 2 stages
  const uint32_t sV = sK + 2 * KV_BYTES_MAX;          // 2 stages
  Control* const ctl = reinterpret_cast<Control*>(smem + Q_BYTES + 4 * KV_BYTES_MAX);
  const uint32_t bar_item_full = smem_u32(&ctl->item_full[0]), bar_item_done = smem_u32(&ctl->item_done[0]);
  const uint32_t bar_q_full = smem_u32(&ctl->q_full[0]), bar_k_full = smem_u32(&ctl->k_full[0]);
  const uint32_t bar_v_full = smem_u32(&ctl->v_full[0]), bar_s_full = smem_u32(&ctl->s_full[0]);
  const uint32_t bar_pv_done = smem_u32(&ctl->pv_done[0]);
  const uint32_t bar_o_free = smem_u32(&ctl->o_free[0]);
  volatile int* const abort_flag = &ctl->abort_flag;
  volatile int* const tile_k0 = ctl->tile_k0;
  volatile ItemSlot* const slots = ctl->slot;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_item_full + 8 * i, 1);
      mbar_init(bar_item_done + 8 * i, kSoftmaxWarps + 1);      // softmax warps + the MMA thread
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_k_full + 8 * i, 1);
      mbar_init(bar_v_full + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_pv_done + 8 * i, 1);
      mbar_init(bar_o_free + 8 * i, kSoftmaxWarps);
    }
    mbar_init(smem_u32(&ctl->drain), 1);
    ctl->abort_flag = 0;
    ctl->p_count[0] = ctl->p_count[1] = 0u;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TmemCols<D>::value);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const long long budget = P.wait_budget;
  const int nt = NT > 0 ? NT : P.nt;
  const uint32_t kv_tile_bytes = (uint32_t)nt * D * 2u;
  const uint32_t kv_panel_bytes = (uint32_t)nt * 128u;

  if (warp == kProducerWarp) {
    // =============================== work fetch + TMA producer ===============================
    const ItemRecord* const records = reinterpret_cast<const ItemRecord*>(P.ws.items);
    unsigned long long* const cursor = reinterpret_cast<unsigned long long*>(P.ws.cursor);
    int I = 0, Iq = 0, T = 0;
    bool ok = P.debug_stall == 0;
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

      // Q has one buffer: the previous item's last S (tile T-1) must be done.  S products complete in
      // order, so this covers tile T-2 (whose K stage the first tile of this item reuses) as well.
      if (T >= 1) ok = warp_wait(bar_of(bar_s_full, T - 1), par_of(T - 1), abort_flag, budget);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(bar_of(bar_q_full, Iq), Q_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(sQ + pn * (128u * 128u), &tm_q, bar_of(bar_q_full, Iq), pn * 64, head0, tile_tok0);
      }
      ++Iq;
      // Active k-blocks of the row, 32 entries at a time and one chunk ahead: bytes of the dense mask row (a warp
      // ballot compacts them), or the entries of the row's CSR list (in-sample block indices, already compact).
      const bool csr = p.csr_ptr != nullptr;
      const int n_src = csr ? rec.count : rec.n_reach;
      const uint8_t* mrow = csr ? nullptr : p.mask + rec.hk * p.mask_s0 + rec.qb * p.mask_s1 + (long long)rec.kb0 * p.mask_s2;
      const int32_t* cidx = csr ? p.csr_idx + rec.csr_begin : nullptr;
      bool bit_next = false;
      int val_next = 0;
      if (csr) val_next = lane < n_src ? cidx[lane] - rec.kb0 : 0;
      else bit_next = lane < n_src && mrow[(long long)lane * p.mask_s2] != 0;
      for (int base = 0; base < n_src && ok; base += 32) {
        uint32_t bal;
        const int val_cur = val_next;
        {                                                   // entries of the next chunk, one chunk ahead
          const int jn = base + 32 + lane;
          if (csr) {
            const int n = n_src - base;
            bal = n >= 32 ? 0xffffffffu : (1u << n) - 1u;
            val_next = jn < n_src ? cidx[jn] - rec.kb0 : 0;
          } else {
            bal = __ballot_sync(0xffffffffu, bit_next);
            bit_next = jn < n_src && mrow[(long long)jn * p.mask_s2] != 0;
          }
        }
        while (bal != 0 && ok) {
          const int pos = __ffs(bal) - 1;
          bal &= bal - 1;
          const int jj = csr ? __shfl_sync(0xffffffffu, val_cur, pos) : base + pos;
          const int blk_k0 = jj * p.kbs;
          for (int sub = 0; sub < P.n_sub && ok; ++sub) {
            const int k0 = blk_k0 + sub * nt;
            if (k0 >= rec.k_len) break;
            if (T >= 2) ok = warp_wait(bar_of(bar_s_full, T), par_of(T - 2), abort_flag, budget);
            if (!ok) break;
            if (lane == 0) {
              tile_k0[T & 3] = k0;
              __threadfence_block();
              mbar_arrive_expect_tx(bar_of(bar_k_full, T), kv_tile_bytes);
#pragma unroll
              for (int pn = 0; pn < PANELS; ++pn)
                tma_load_3d(sK + (T & 1) * KV_BYTES_MAX + pn * kv_panel_bytes, &tm_k, bar_of(bar_k_full, T), pn * 64, rec.hk, rec.k_begin + k0);
              if (TRACE) stamp(P.trace, T, 0);
            }
            // V stage T & 1 is free once the P V product of tile T-2 is done
            if (T >= 2) ok = warp_wait(bar_of(bar_pv_done, T), par_of(T - 2), abort_flag, budget);
            if (!ok) break;
            if (lane == 0) {
              mbar_arrive_expect_tx(bar_of(bar_v_full, T), kv_tile_bytes);
#pragma unroll
              for (int pn = 0; pn < PANELS; ++pn)
                tma_load_3d(sV + (T & 1) * KV_BYTES_MAX + pn * kv_panel_bytes, &tm_v, bar_of(bar_v_full, T), pn * 64, rec.hk, rec.k_begin + k0);
              if (TRACE) stamp(P.trace, T, 1);
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
    // One thread issues every tcgen05.mma of the CTA in the order S(0), S(1), PV(0), S(2), PV(1), S(3), ...
    // S(t+2) goes into the buffer that P(t) occupies and is issued right behind PV(t) without waiting for
    // PV(t) to complete: instructions of one thread execute in issue order, so PV(t) has read P(t) before
    // S(t+2) writes.  The thread polls with non-blocking probes and issues whichever of "next P V" / "next
    // S" has its inputs ready; a clock budget bounds the loop.
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc(BF16, false, false, 128, nt);
      const uint32_t idesc_pv = make_idesc(BF16, false, true, 128, D);
      const int ksteps = nt >> 4;
      const uint32_t desc_hi = smem_desc_hi(1024u);
      const uint32_t kpanel_units = kv_panel_bytes >> 4;
      // Q and K are K-major: 16 head dims further = 32 bytes = 2 descriptor units inside a 64-dim panel.
      // V is MN-major: 16 keys further = 2048 bytes = 128 units.  P: 8 TMEM columns per 16 keys.
      uint64_t qd[D / 16], kd0[D / 16], kd1[D / 16], vd0[4], vd1[4];
      uint32_t pa0[4], pa1[4];
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t ko = (uint32_t)(ks >> 2) * kpanel_units + (uint32_t)(ks & 3) * 2u;
        const uint32_t qo = (uint32_t)(ks >> 2) * 1024u + (uint32_t)(ks & 3) * 2u;
        qd[ks] = smem_desc_join(smem_desc_lo(sQ, 16u) + qo, desc_hi);
        kd0[ks] = smem_desc_join(smem_desc_lo(sK, 16u) + ko, desc_hi);
        kd1[ks] = smem_desc_join(smem_desc_lo(sK + KV_BYTES_MAX, 16u) + ko, desc_hi);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        vd0[ks] = smem_desc_join(smem_desc_lo(sV, kv_panel_bytes) + (uint32_t)ks * 128u, desc_hi);
        vd1[ks] = smem_desc_join(smem_desc_lo(sV + KV_BYTES_MAX, kv_panel_bytes) + (uint32_t)ks * 128u, desc_hi);
        pa0[ks] = tmem_base + (uint32_t)ks * 8u;
        pa1[ks] = tmem_base + kSStride + (uint32_t)ks * 8u;
      }
      const uint32_t tO = tmem_base + kTmemOCol;
      // S side: item qI (count of published items), its tiles left, number of items with tiles so far, next tile
      int qI = 0, q_left = 0, qIq = 0, qT = 0;
      bool q_have = false, q_first = false, finished = false;
      // P V side: the items whose tiles are in flight, per tile "first of its item" / "last of its item"
      int pT = 0;                    // next tile to issue P V for (pT <= qT <= pT + 2)
      int pIq = 0;                   // items with tiles whose first P V has been issued
      // per in-flight tile (tile & 1): packed flags  bit 0 first of its item, bit 1 last of its item, bits 2.. item number
      int fl0 = 0, fl1 = 0;
      bool v_landed = false, p_seen = false;
      unsigned idle = 0u;
      long long t_idle = 0;
      while (true) {
        bool progress = false;
        if (!q_have && !finished && mbar_test(bar_of(bar_item_full, qI), par_of(qI))) {
          const int n_tiles = slots[qI & 1].n_tiles;
          if (n_tiles < 0) {
            finished = true;
          } else if (n_tiles == 0) {
            mbar_arrive(bar_of(bar_item_done, qI));
            ++qI;
          } else {
            q_have = true;
            q_first = true;
            q_left = n_tiles;
          }
          progress = true;
        }
        if (pT < qT) {
          // one probe per idle turn in the steady state: that V(pT) has landed is looked up once and remembered
          if (!v_landed) {
            v_landed = mbar_test(bar_of(bar_v_full, pT), par_of(pT));
            if (TRACE && v_landed) stamp(P.trace, pT, 18);
          }
          const bool p_there = *(volatile unsigned*)&ctl->p_count[pT & 1] >= (unsigned)kSoftmaxWarps * ((unsigned)(pT >> 1) + 1u);
          if (TRACE && !p_seen && p_there) {
            p_seen = true;
            stamp(P.trace, pT, 17);
          }
          bool ready = v_landed && p_there;
          // the first P V of an item overwrites O: the epilogue of the previous item must have read it
          const int fl = (pT & 1) ? fl1 : fl0;
          if (ready && (fl & 1) && pIq >= 1) ready = mbar_test(bar_of(bar_o_free, pIq - 1), par_of(pIq - 1));
          if (ready) {
            // No tcgen05.fence::after_thread_sync here in the shipped build: P(t) is complete in TMEM before
            // the counter can reach its value (tcgen05.wait::st precedes the increments), and the MMA is issued after
            // that was observed.  HBSA_STRICT_TCGEN05 builds execute the fence; the two builds must agree bit for bit.
#ifdef HBSA_STRICT_TCGEN05
            tc_fence_after();
#endif
            if (TRACE) stamp(P.trace, pT, 4);
            if (pT & 1) issue_pv(ksteps, tO, pa1, vd1, idesc_pv, (fl & 1) != 0);
            else issue_pv(ksteps, tO, pa0, vd0, idesc_pv, (fl & 1) != 0);
            tc_commit(bar_of(bar_pv_done, pT));
            if (TRACE) stamp(P.trace, pT, 5);
            if (fl & 1) ++pIq;
            if (fl & 2) mbar_arrive(bar_of(bar_item_done, fl >> 2));       // through with the item
            ++pT;
            v_landed = false;
            p_seen = false;
            progress = true;
          }
        }
        if (q_have && qT < pT + 2) {
          bool ready = mbar_test(bar_of(bar_k_full, qT), par_of(qT));
          if (ready && q_first) ready = mbar_test(bar_of(bar_q_full, qIq), par_of(qIq));
#ifdef HBSA_STRICT_TCGEN05
          // S(t) overwrites the columns of P(t-2): wait until P V(t-2) has completed instead of relying on the
          // issue order of this thread, and fence after every observation
          if (ready && qT >= 2) ready = mbar_test(bar_of(bar_pv_done, qT - 2), par_of(qT - 2));
          if (ready) tc_fence_after();
#endif
          if (ready) {
            if (TRACE) stamp(P.trace, qT, 2);
            const uint32_t tSb = tmem_base + (uint32_t)(qT & 1) * kSStride;
            if (qT & 1) issue_qk<D / 16>(tSb, qd, kd1, idesc_qk);
            else issue_qk<D / 16>(tSb, qd, kd0, idesc_qk);
            tc_commit(bar_of(bar_s_full, qT));
            if (TRACE) stamp(P.trace, qT, 3);
            const int fl_new = (q_first ? 1 : 0) | (q_left == 1 ? 2 : 0) | (qI << 2);
            if (qT & 1) fl1 = fl_new; else fl0 = fl_new;
            ++qT;
            if (q_first) ++qIq;
            q_first = false;
            if (--q_left == 0) {
              ++qI;
              q_have = false;
            }
            progress = true;
          }
        }
        if (finished && pT == qT) break;
        if (progress) {
          idle = 0;
        } else if ((++idle & 63u) == 0u) {                  // give-up checks on one idle turn in 64: they cost as much as a probe
          if (*abort_flag) break;
          const long long now = clock64();
          if (idle == 64u) t_idle = now;
          else if (now - t_idle > budget) { *abort_flag = 1; break; }
        }
      }
      // Whatever this thread has issued completes before the CTA gives its tensor memory back, also when it gave up
      // (bounded by the clock alone: the abort flag is already set then).
      tc_commit(smem_u32(&ctl->drain));
      mbar_wait_clock(smem_u32(&ctl->drain), 0u, budget);
    }
    __syncwarp();
  } else {
    // =============================== softmax + epilogue ===============================
    const int row = tid;                             // 0..127: row of the M tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const int my_nc = nt;                            // columns of a tile: 16, 32, 48 or 64
    const uint32_t tOmine = tmem_base + kTmemOCol + lane_off;
    const float scale_log2 = P.scale_log2;
    int I = 0, Iq = 0, T = 0;
    bool ok = true;
    while (ok) {
      ok = warp_wait(bar_of(bar_item_full, I), par_of(I), abort_flag, budget);
      if (!ok) break;
      const int n_tiles = slots[I & 1].n_tiles;
      if (n_tiles < 0) break;
      const int tile_tok0 = slots[I & 1].tile_tok0, head0 = slots[I & 1].head0, q_end = slots[I & 1].q_end;
      if (n_tiles == 0) {
        // No active k-block: the rows are exact zeros (fwd_triton_fix_tile_size.py:189).
        const int r_tok = tile_tok0 + (row >> P.gp_shift);
        if (r_tok < q_end) {
          uint4* dst = reinterpret_cast<uint4*>(o_base + r_tok * P.o_s0 + (head0 + (row & (P.gp - 1))) * P.o_s1);
#pragma unroll
          for (int i = 0; i < D / 8; ++i)
            if (i * 8 < p.headdim) dst[i] = make_uint4(0, 0, 0, 0);
          if (P.lse != nullptr) P.lse[(long long)r_tok * p.nhead_q + head0 + (row & (P.gp - 1))] = -INFINITY;
        }
      } else {
        int limit_row = slots[I & 1].k_len - 1;
        if (p.causal) limit_row = min(limit_row, slots[I & 1].qi0 + (row >> P.gp_shift) + slots[I & 1].off);
        float m_ref = -INFINITY, l = 0.f;
        if (TRACE && tid == 0) stamp(P.trace, T, 10);
        for (int t = 0; t < n_tiles && ok; ++t, ++T) {
          ok = warp_wait(bar_of(bar_s_full, T), par_of(T), abort_flag, budget);
          if (!ok) break;
          tc_fence_after();
          if (TRACE && tid == 0) stamp(P.trace, T, 6);
          const int col_limit = limit_row - tile_k0[T & 3];            // tile columns <= col_limit are valid
          const uint32_t tSmine = tmem_base + (uint32_t)(T & 1) * kSStride + lane_off;

          // ---- this thread's row of S, all in registers.  The first 16 columns are awaited alone so that
          //      work on them overlaps the TMEM latency of the rest.
          uint32_t r[64];
          const bool edge = col_limit < my_nc - 1;      // tile on the causal diagonal or at the ragged end of the sample
          tmem_ld16(tSmine, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
          tmem_wait_ld();
#pragma unroll
          for (int j = 1; j < 4; ++j)
            if (my_nc > 16 * j) tmem_ld16(tSmine + 16 * j, *reinterpret_cast<uint32_t(*)[16]>(&r[16 * j]));
          if (TRACE && tid == 0) stamp(P.trace, T, 12);

          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          bool exact = t == 0;                           // first tile of the item: the maximum must come first
          if (!exact) {
            // Optimistic pass: exponentials against the reference maximum of the previous tiles (any reference
            // gives the same softmax; the reference only has to keep P in range).  If the tile turns out to be
            // out of range, the exact pass below redoes it.
            const float neg_m0 = m_ref == -INFINITY ? 0.f : -m_ref;
            // With the tile width fixed at compile time, tiles without masked columns (all but those on the causal
            // diagonal or at the ragged end of a sample) take a copy of the loop that has no per-group branch; the
            // test is warp-uniform because the TMEM stores are warp-wide instructions.
            if (NT > 0 && !__any_sync(0xffffffffu, edge)) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (my_nc > 16 * j) {
                  if (j == 1) tmem_wait_ld();
                  uint32_t pk[8];
                  exp16<BF16>(&r[16 * j], pk, scale_log2, neg_m0, sum);
                  tmem_st8(tSmine + 8 * j, pk);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (my_nc > 16 * j) {
                  if (j == 1) tmem_wait_ld();
                  if (edge) {
#pragma unroll
                    for (int i = 16 * j; i < 16 * j + 16; ++i)
                      if (i > col_limit) r[i] = 0xff800000u;               // -inf: exp2 makes it an exact 0
                  }
                  uint32_t pk[8];
                  exp16<BF16>(&r[16 * j], pk, scale_log2, neg_m0, sum);
                  tmem_st8(tSmine + 8 * j, pk);
                }
              }
            }
            if (my_nc <= 16) tmem_wait_ld();
            // Whether the reference is stale is read off the tile's row sum, which is there anyway: P >= 0, so no P
            // exceeds it, and a sum of at most 2^14 keeps every P far inside the range of both 16-bit formats (an
            // overflowed exponential makes the sum infinite).  The row maximum itself is only computed on that (rare)
            // path.  Rows without a reference yet take it as well.
            const float tile_sum = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            bool need = !(tile_sum <= 16384.f) || m_ref == -INFINITY;
            if (TRACE && tid == 0) stamp(P.trace, T, 7);
            if (__any_sync(0xffffffffu, need)) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (my_nc > 16 * j) max16(&r[16 * j], mx4);
              const float mx_s = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale > 0 keeps the order
              need = mx_s > m_ref + kRescaleThreshold;
              if (__any_sync(0xffffffffu, need)) {       // (a row without reference whose tile is all masked needs nothing)
                // O and l move to the new reference maximum; needs the P V product of the previous tile
                ok = warp_wait(bar_of(bar_pv_done, T - 1), par_of(T - 1), abort_flag, budget);
                if (!ok) break;
                tc_fence_after();
                const float alpha = need ? ex2_approx(m_ref - mx_s) : 1.f;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                  uint32_t o[32];
                  tmem_ld32(tOmine + c0, o);
                  tmem_wait_ld();
#pragma unroll
                  for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                  tmem_st32(tOmine + c0, o);
                }
                tmem_wait_st();
                l *= alpha;
                if (need) m_ref = mx_s;
                exact = true;                            // P of this tile is recomputed against the new reference
                sum[0] = sum[1] = sum[2] = sum[3] = 0.f;
              }
            }
          } else {
            tmem_wait_ld();
            if (edge) {
#pragma unroll
              for (int i = 0; i < 64; ++i)
                if (i > col_limit) r[i] = 0xff800000u;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (my_nc > 16 * j) max16(&r[16 * j], mx4);
            m_ref = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            if (TRACE && tid == 0) stamp(P.trace, T, 7);
          }
          if (exact) {
            // ---- P = exp2(S * scale - m) packed to 16 bit over the first half of the S columns, row sum
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (my_nc > 16 * j) {
                uint32_t pk[8];
                exp16<BF16>(&r[16 * j], pk, scale_log2, neg_m, sum);
                tmem_st8(tSmine + 8 * j, pk);
              }
            }
          }
          l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
          tmem_wait_st();
          tc_fence_before();
          if (TRACE && tid == 0) stamp(P.trace, T, 8);
          __syncwarp();
          if (lane == 0) {                                               // one arrival per warp, on a plain shared-memory counter
            __threadfence_block();
            atomicAdd(&ctl->p_count[T & 1], 1u);
          }
          if (TRACE && lane == 0) stamp(P.trace, T, warp == 0 ? 9 : 13 + warp);        // slots 9, 14, 15, 16: arrival of warps 0..3
        }
        if (!ok) break;

        // ---- epilogue: O / l -> global; rows past the q-block end are dropped, rows that saw no key are zeros
        if (TRACE && tid == 0) stamp(P.trace, T - 1, 13);
        const bool live = l > 0.f;
        const float inv = live ? 1.f / l : 0.f;
        const uint64_t inv2 = pack_f32x2(inv, inv);
        if (P.lse != nullptr) {
          // ln sum exp of the row's scaled scores = ln 2 * (reference + log2 l), whatever reference was used
          const int r_tok = tile_tok0 + (tid >> P.gp_shift);
          if (r_tok < q_end)
            P.lse[(long long)r_tok * p.nhead_q + head0 + (tid & (P.gp - 1))] = live ? 0.6931471805599453f * (m_ref + log2f(l)) : -INFINITY;
        }
        ok = warp_wait(bar_of(bar_pv_done, T - 1), par_of(T - 1), abort_flag, budget);
        if (!ok) break;
        tc_fence_after();
        if (TRACE && tid == 0) stamp(P.trace, T - 1, 22);
        // 64 columns of O per TMEM round trip; every thread writes its own row, 32 bytes (one full sector) per store
        // when the output rows are 32-byte aligned, 16 bytes otherwise
        const int r_tok_o = tile_tok0 + (tid >> P.gp_shift);
        const bool store_row = r_tok_o < q_end;
        const bool fast_store = store_row && P.o_vec32 != 0 && p.headdim == D;
        OutT* const orow = o_base + r_tok_o * P.o_s0 + (head0 + (tid & (P.gp - 1))) * P.o_s1;
#pragma unroll
        for (int cb = 0; cb < D; cb += 64) {
          uint32_t oa[64];
          tmem_ld32(tOmine + cb, *reinterpret_cast<uint32_t(*)[32]>(&oa[0]));
          tmem_ld32(tOmine + cb + 32, *reinterpret_cast<uint32_t(*)[32]>(&oa[32]));
          tmem_wait_ld();
          if (cb + 64 >= D) {
            tc_fence_before();                                             // O is in registers: the next item may overwrite it
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_of(bar_o_free, Iq));
            if (TRACE && tid == 0) stamp(P.trace, T - 1, 23);
          }
          if (fast_store) {
            // the common case (row inside the q-block, 32-byte aligned rows, no padded columns): no branch per group
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
              uint32_t w[8];
#pragma unroll
              for (int e = 0; e < 16; e += 2) {
                float y0, y1;
                unpack_f32x2(mul_f32x2(pack_b32x2(oa[c0 + e], oa[c0 + e + 1]), inv2), y0, y1);
                w[e >> 1] = live ? pack2<BF16>(y0, y1) : 0u;
              }
              st_global_v8(orow + cb + c0, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
            }
            continue;
          }
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              float y0, y1;
              unpack_f32x2(mul_f32x2(pack_b32x2(oa[c0 + e], oa[c0 + e + 1]), inv2), y0, y1);
              w[e >> 1] = live ? pack2<BF16>(y0, y1) : 0u;
            }
            // columns at and past the real head dimension are padding (zeros); it is a multiple of 8
            if (store_row && cb + c0 < p.headdim) {
              if (cb + c0 + 8 >= p.headdim) {
                *reinterpret_cast<uint4*>(orow + cb + c0) = make_uint4(w[0], w[1], w[2], w[3]);
              } else if (P.o_vec32) {
                st_global_v8(orow + cb + c0, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
              } else {
                *reinterpret_cast<uint4*>(orow + cb + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(orow + cb + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
              }
            }
          }
        }
        if (TRACE && tid == 0) stamp(P.trace, T - 1, 11);
        ++Iq;
      }
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
    tmem_dealloc(tmem_base, TmemCols<D>::value);
  }
  if (tid == 0 && ctl->abort_flag) {
    atomicExch(&P.ws.status[0], HBSA_STATUS_WAIT_LIMIT);
    P.ws.status[3] = (int)blockIdx.x;
  }
  // The last CTA to leave rewinds the work cursor, so that the same schedule can drive the next launch
  // (every CTA is past its last fetch by the time it gets here).  Word 2 of the cursor block counts the leavers.
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(reinterpret_cast<unsigned int*>(P.ws.cursor) + 2, 1u) == gridDim.x - 1) {
      *reinterpret_cast<volatile unsigned long long*>(P.ws.cursor) = 0ull;
      reinterpret_cast<volatile unsigned int*>(P.ws.cursor)[2] = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
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
long long g_wait_budget = 4000000000ll;   // clock64 ticks a wait inside the kernel may take (about two seconds)
int g_debug_stall = 0;

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

void sm100_set_wait_budget(long long clocks, int stall_producer) {
  g_wait_budget = clocks > 0 ? clocks : 4000000000ll;
  g_debug_stall = stall_producer ? 1 : 0;
}
void sm100_set_trace(long long* device_buffer) { g_trace = device_buffer; }
size_t sm100_trace_bytes() { return ((size_t)kTraceTiles * kTraceSlots + 2 * kTraceCtas) * sizeof(long long); }

int sm100_kv_tile_rows(int kbs) {
  if (kbs <= kTileRowsMax) return kbs;
  for (int nt = kTileRowsMax; nt >= 16; nt -= 16)
    if (kbs % nt == 0) return nt;
  return 16;
}

const char* sm100_ineligible_reason(const hbsa_forward_args& a, float scale) {
  if (a.dtype != HBSA_DTYPE_BF16 && a.dtype != HBSA_DTYPE_F16) return "dtype is not bf16/fp16";
  if (a.headdim % 8 != 0 || a.headdim < 16 || a.headdim > 256) return "headdim is not a multiple of 8 between 16 and 256";
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
  P.lse = a.lse;
  P.total_q = a.total_q;
  P.o_s0 = a.o_stride[0];
  P.o_s1 = a.o_stride[1];
  P.nt = sm100_kv_tile_rows(p.kbs);
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
  P.wait_budget = g_wait_budget;
  P.o_vec32 = ((uintptr_t)a.o % 32 == 0 && (a.o_stride[0] * 2) % 32 == 0 && (a.o_stride[1] * 2) % 32 == 0) ? 1 : 0;
  P.debug_stall = g_debug_stall;
  P.trace = g_trace;

  P.total_items = (long long)p.nhead_k * p.num_q_block * P.items_per_row;
  if (P.total_items <= 0) { *err_text = "no work items"; return HBSA_ERR_SHAPE; }
  // two persistent CTAs per SM; one above 128 head dimensions (O alone takes 256 of the SM's 512 TMEM columns, the
  // tiles 192 KB of its shared memory)
  const long long resident = (p.headdim > 128 ? 1ll : 2ll) * sm_count();
  const unsigned grid = (unsigned)(P.total_items < resident ? P.total_items : resident);

  CUtensorMap tq, tk, tv;
  if (!encode_map(fn, &tq, bf16, a.q, p.headdim, p.nhead_q, a.total_q, a.q_stride[0], a.q_stride[1], gp, P.tt) ||
      !encode_map(fn, &tk, bf16, a.k, p.headdim, p.nhead_k, a.total_k, a.k_stride[0], a.k_stride[1], 1, P.nt) ||
      !encode_map(fn, &tv, bf16, a.v, p.headdim, p.nhead_k, a.total_k, a.v_stride[0], a.v_stride[1], 1, P.nt)) {
    *err_text = "cuTensorMapEncodeTiled rejected a q/k/v layout";
    return HBSA_ERR_UNSUPPORTED;
  }

  // Head dimensions other than 64 and 128 run on the next larger of the two: the TMA boxes reach past the tensors'
  // innermost extent, the hardware fills those columns of Q, K and V with zeros (so S is exact and the surplus
  // columns of O are zeros), and the epilogue stores the real columns only.
  const int d_tile = p.headdim <= 64 ? 64 : p.headdim <= 128 ? 128 : 256;
  const size_t smem = (128u + 4u * (size_t)kTileRowsMax) * (size_t)d_tile * 2u + sizeof(Control) + 1024u;
  cudaError_t e = cudaSuccess;
#define HBSA_LAUNCH_SM100(D_, BF_, TR_, NT_)                                                              \
  do {                                                                                                   \
    e = cudaFuncSetAttribute(fwd_sm100_kernel<D_, BF_, TR_, NT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) {                                                                              \
      fwd_sm100_kernel<D_, BF_, TR_, NT_><<<grid, kThreads, smem, stream>>>(tq, tk, tv, P);              \
      e = cudaGetLastError();                                                                            \
    }                                                                                                    \
  } while (0)
#define HBSA_LAUNCH_SM100_T(D_, BF_)                                                                      \
  do {                                                                                                   \
    if (P.trace != nullptr) HBSA_LAUNCH_SM100(D_, BF_, true, 0);                                         \
    else if (P.nt == 64) HBSA_LAUNCH_SM100(D_, BF_, false, 64);                                          \
    else HBSA_LAUNCH_SM100(D_, BF_, false, 0);                                                           \
  } while (0)
  if (d_tile == 256) { if (bf16) HBSA_LAUNCH_SM100_T(256, true); else HBSA_LAUNCH_SM100_T(256, false); }
  else if (d_tile == 128) { if (bf16) HBSA_LAUNCH_SM100_T(128, true); else HBSA_LAUNCH_SM100_T(128, false); }
  else { if (bf16) HBSA_LAUNCH_SM100_T(64, true); else HBSA_LAUNCH_SM100_T(64, false); }
#undef HBSA_LAUNCH_SM100_T
#undef HBSA_LAUNCH_SM100
  if (e != cudaSuccess) { *err_text = cudaGetErrorString(e); return (int)e; }
  return 0;
}

}  // namespace hbsa
