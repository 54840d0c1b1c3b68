// Block-sparse attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces the two Triton kernels of the reference (fwd_triton_fix_tile_size.py:30-212,
// fwd_triton_auto_tile_size.py:76-251).  Differences of design, not of result:
//
//  * A work item is one 128-row M tile of one (kv-head, q-block): `TT = 128 / GP` tokens times
//    `GP` q-heads of the GQA group packed into the MMA M dimension, so that one K/V tile fetch
//    serves GP heads (the reference runs one program per q-head and re-reads K/V per head).
//  * One persistent CTA per SM works on TWO independent items at a time ("lanes" A and B), each with
//    its own Q tile, its own S and O accumulators in TMEM and its own four softmax warps.  While the
//    softmax warps of one lane turn S into P, the tensor pipe runs the products of the other lane,
//    so the two latency chains S -> softmax -> P V interleave on one tensor pipe that a single thread
//    feeds in a fixed order.  Items come from an atomic cursor over the ItemRecord table the schedule
//    kernels wrote.
//  * Only mask-active k-blocks are touched: the producer warp compacts the mask row with warp
//    ballots and issues TMA loads of exactly those K/V tiles (up to 128 rows each) into one ring of
//    shared-memory slots that both lanes share, in the order the MMA thread consumes them (the
//    reference loops over all k-blocks of the sample and polls the mask byte,
//    fwd_triton_fix_tile_size.py:117-124).
//  * S = Q K^T is one M128 x N<=128 tcgen05.mma chain per K tile; O += P V is issued in two groups of
//    up to 64 keys, so the first group runs while the softmax warps are still in the exponentials of
//    the second 64 columns.  P (in the input dtype, as at fwd_triton_fix_tile_size.py:187) is written
//    back into TMEM over S columns that were already read and consumed as the A operand of the
//    second MMA, so it never touches shared memory.  Because tcgen05.mma instructions of one thread
//    execute in issue order, S(t+1) of a lane is issued right behind P V(t) into the columns P(t)
//    occupies without waiting for P V(t) to complete (HBSA_STRICT_TCGEN05 builds wait and fence
//    instead; they exist to check this ordering).
//  * Online softmax in registers, one thread per row, 64 columns at a time: in-place -inf masking on
//    diagonal / ragged tiles, exp2 with the scale folded in, fp32 row sum; no shuffles and no
//    shared-memory exchange.  The exponentials run against the reference maximum of the previous
//    columns; whether that reference is stale is read off the packed P itself, and only then is the
//    running output rescaled in TMEM and the 64 columns redone exactly from registers.
//  * The last CTA to leave rewinds the work cursor, so one schedule serves any number of launches.
//    With `lse` set, ln sum exp of every row goes out beside O.
//
// Warp roles (320 threads): warps 0-3 softmax + epilogue of lane A, warps 4-7 of lane B (TMEM lane
// quarter = warp id % 4), warp 8 TMEM allocator + MMA issuer, warp 9 work fetch + TMA producer.
// TMEM (512 columns): S_A [0,128), S_B [128,256), O_A [256,256+D), O_B [256+D,256+2D).
//
// mbarriers.  Per lane: T counts K/V tiles, I published items, Iq those of them that have tiles.  A waiter
// for the c-th completion of a barrier uses parity c & 1, which is only sound while the barrier is at most one
// completion ahead of what the waiter looks for.  That holds for every single-entry barrier below because its
// waiter observes each completion before the next one can happen; barriers whose waiters look only now and
// then (item_*, pv_done) are two-entry arrays indexed by the low bit of the count, with parity (count >> 1) & 1.
//   ring_full / ring_empty [slot]: TMA bytes landed / the product that read the slot is done
//   s_full [lane]: S = Q K^T done                   p_full [lane][half]: P of 64 columns written
//   pv_done [lane][half][2]: O += P V of the half done   q_full / q_free [lane]: Q landed / last S of the item done
//   o_free [lane]: epilogue has read O out of TMEM  item_full / item_done [lane][2]: item slot written / left
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

constexpr int kThreads = 320;
constexpr int kLaneWarps = 4;         // softmax warps per lane
constexpr int kMmaWarp = 8;
constexpr int kProducerWarp = 9;
constexpr int kTileRowsMax = 128;     // rows of a K/V tile
constexpr int kSubCols = 64;          // columns the softmax handles at a time
constexpr int kTmemCols = 512;
constexpr uint32_t kTmemSStride = 128u;
constexpr uint32_t kTmemOBase = 256u;
constexpr int kMaxSlots = 8;          // K/V ring
constexpr int kMinSlots = 4;
constexpr int kTileInfo = 8;          // per-lane ring of tile start columns
constexpr float kRescaleThreshold = 8.0f;   // log2 units
constexpr size_t kSmemLimit = 232448; // dynamic shared memory a CTA may opt into on sm_100

struct Sm100Params {
  Problem p;
  Workspace ws;
  void* o;
  long long o_s0, o_s1;        // elements
  float* lse;                  // NULL or [total_q, nhead_q]: natural-log sum of exponentials per row
  int total_q;
  int nt;                      // rows of one K/V tile (multiple of 16, <= 128)
  int n_sub;                   // K/V tiles per k-block
  int gp, gp_shift;            // q-heads packed into one M tile
  int n_head_sub;              // group / gp
  int tt;                      // tokens per M tile = 128 / gp
  int tiles_per_qblock;
  int items_per_row;           // n_head_sub * tiles_per_qblock
  long long total_items;       // rows * items_per_row
  int n_slots;                 // K/V ring slots
  uint32_t slot_bytes;
  int o_vec32;                 // output rows are 32-byte aligned: 256-bit stores
  int debug_stall;             // debugging aid: the producer publishes nothing, every wait runs out
  float scale_log2;
  long long wait_budget;       // clock64 ticks
  long long* trace;            // debugging aid: clock64 stamps of CTA 0 (NULL in normal use)
};

// Debugging aid.  While a trace buffer is set, four threads of CTA 0 (the MMA thread, the first thread of each
// lane's softmax warps, the first thread of the producer warp) write (clock64 << 8 | code) stamps of their
// pipeline events into their own region of kTraceCap entries; entry 0 of a region holds the number of stamps.
// The shipped instantiation carries no stamp code at all.
constexpr int kTraceCap = 8192;
constexpr int kTraceRegions = 4;
template <bool TRACE>
struct Tracer {
  long long* base;
  int n;
  __device__ __forceinline__ void init(long long* buf, int region, bool mine) {
    base = (TRACE && buf != nullptr && mine && blockIdx.x == 0) ? buf + (size_t)region * kTraceCap : nullptr;
    n = 1;
  }
  __device__ __forceinline__ void put(int code) {
    if (TRACE) {
      if (base != nullptr && n < kTraceCap) base[n++] = (clock64() << 8) | (long long)code;
    }
  }
  __device__ __forceinline__ void done() {
    if (TRACE) {
      if (base != nullptr) base[0] = n - 1;
    }
  }
};

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
  unsigned long long ring_full[kMaxSlots], ring_empty[kMaxSlots];
  unsigned long long item_full[2][2], item_done[2][2];
  unsigned long long q_full[2], q_free[2], s_full[2], p_full[2][2], pv_done[2][2][2], o_free[2];
  unsigned long long drain;
  uint32_t tmem_base;
  int abort_flag;
  int tile_k0[2][kTileInfo];
  ItemSlot slot[2][2];
};

// Compile-time tuning knobs of the softmax threads (see exp16):
//   HBSA_POLY_PAIRS  of every 8 column pairs, how many take their exponentials from a polynomial on the FMA pipe
//                    instead of the exp unit (0..8); only bf16/fp16 tiles without masked columns use it
//   HBSA_ALU_PACK    1: fp32 -> bf16 pairs are packed with integer adds and a byte permute instead of cvt
#ifndef HBSA_POLY_PAIRS
#define HBSA_POLY_PAIRS 0
#endif
#ifndef HBSA_ALU_PACK
#define HBSA_ALU_PACK 0
#endif

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// P >= 0 and finite-or-inf: rounding to bf16 is "add half an ulp of the kept part, keep the upper 16 bits" (ties go
// up instead of to even, one ulp apart once in 2^16 values).  The conversion instruction shares the exp unit, which is
// the pipe the softmax threads saturate; these three run on the integer pipe.
template <bool BF16> __device__ __forceinline__ uint32_t pack2_p(float lo, float hi) {
  if (BF16 && HBSA_ALU_PACK)
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
  return pack2<BF16>(lo, hi);
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
// 2^x for two values by polynomial on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f from a
// cubic (relative error 7.5e-5, far below the 2^-9 of the 16-bit P it is rounded to); n goes straight into the
// exponent field.  x is clamped to [-126, 255]: below, the result is a tiny normal number; above 128 the exponent
// overflows into a bit pattern that, read as an unsigned 16-bit float, is larger than any legal P - exactly what
// the staleness check of the caller looks for.
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& p0, float& p1) {
  float x0, x1;
  ptx::unpack_f32x2(x2, x0, x1);
  x0 = fminf(fmaxf(x0, -126.f), 255.f);
  x1 = fminf(fmaxf(x1, -126.f), 255.f);
  const uint64_t xc = ptx::pack_f32x2(x0, x1);
  const uint64_t magic = ptx::pack_f32x2(12582912.f, 12582912.f);          // 1.5 * 2^23: the sum's low mantissa bits are round(x)
  const uint64_t t = ptx::add_f32x2(xc, magic);
  const uint64_t n = ptx::add_f32x2(t, ptx::pack_f32x2(-12582912.f, -12582912.f));
  const uint64_t f = ptx::fma_f32x2(n, ptx::pack_f32x2(-1.f, -1.f), xc);
  uint64_t q = ptx::fma_f32x2(f, ptx::pack_f32x2(0.05517164617776871f, 0.05517164617776871f), ptx::pack_f32x2(0.2426111251115799f, 0.2426111251115799f));
  q = ptx::fma_f32x2(q, f, ptx::pack_f32x2(0.6932609677314758f, 0.6932609677314758f));
  q = ptx::fma_f32x2(q, f, ptx::pack_f32x2(0.9999280571937561f, 0.9999280571937561f));
  float q0, q1, t0, t1;
  ptx::unpack_f32x2(q, q0, q1);
  ptx::unpack_f32x2(t, t0, t1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// P = exp2(S * scale - m) for 16 columns, packed to 16-bit pairs; four independent partial row sums.
// The scale-and-shift and the sums use the two-wide fp32 instructions: same FMA-pipe time, half the
// issue slots.  POLY of the 8 column pairs take the polynomial (callers pass 0 for tiles with masked columns:
// -inf must come out as an exact zero).
template <bool BF16, int POLY>
__device__ __forceinline__ void exp16(const uint32_t* r, uint32_t (&pk)[8], float scale_log2, float neg_m, float (&sum)[4]) {
  const uint64_t scale2 = ptx::pack_f32x2(scale_log2, scale_log2), neg_m2 = ptx::pack_f32x2(neg_m, neg_m);
  uint64_t sa = ptx::pack_f32x2(sum[0], sum[2]), sb = ptx::pack_f32x2(sum[1], sum[3]);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const int q = i >> 1;
    const uint64_t x2 = ptx::fma_f32x2(ptx::pack_b32x2(r[i], r[i + 1]), scale2, neg_m2);
    float p0, p1;
    if (((q + 1) * POLY) / 8 > (q * POLY) / 8) {
      exp2_poly2(x2, p0, p1);
    } else {
      float x0, x1;
      ptx::unpack_f32x2(x2, x0, x1);
      p0 = ptx::ex2_approx(x0);
      p1 = ptx::ex2_approx(x1);
    }
    if (q & 1) sb = ptx::add_f32x2(sb, ptx::pack_f32x2(p0, p1));
    else sa = ptx::add_f32x2(sa, ptx::pack_f32x2(p0, p1));
    pk[q] = pack2_p<BF16>(p0, p1);
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
__device__ __forceinline__ uint32_t bar2(uint32_t base, int c) { return base + 8u * (uint32_t)(c & 1); }
__device__ __forceinline__ uint32_t par2(int c) { return (uint32_t)(c >> 1) & 1u; }

// pv_done barrier of (lane, half of the tile) for the lane's tile number T, and the parity to wait for.
__device__ __forceinline__ uint32_t pv_bar(uint32_t base, int L, int h, int T) { return base + 32u * (uint32_t)L + 16u * (uint32_t)h + 8u * (uint32_t)(T & 1); }
__device__ __forceinline__ uint32_t pv_par(int T) { return (uint32_t)(T >> 1) & 1u; }

// Position in the K/V ring: slot index and the parity of its current use.
struct RingPos {
  int slot;
  uint32_t phase;
  __device__ __forceinline__ void advance(int n_slots) {
    if (++slot == n_slots) { slot = 0; phase ^= 1u; }
  }
};

// Per-lane state of the producer warp (all values warp-uniform except bit_next).
struct ProdLane {
  bool done, pend_v;
  int pend_tok;              // global token of the first row of the tile whose V is still to be loaded
  int hk;
  int tiles_left;
  const uint8_t* mrow;       // dense mask: mask row of the item, at the sample's first k-block
  const int32_t* cidx;       // CSR mask: the row's first active entry
  int n_reach, k_begin, k_len, kb0;
  int n_src;                 // entries to scan: causal-reachable k-blocks (dense) or active entries (CSR)
  int base;                  // first entry of the 32-entry chunk `bal` describes
  uint32_t bal;              // active blocks of the chunk not handed out yet
  bool bit_next;             // dense: this lane's mask byte of the chunk after `base`
  int val_cur, val_next;     // CSR: this lane's in-sample k-block index of the chunk at / after `base`
  int blk, sub;              // block being handed out and its next sub-tile
  int I, Iq, T;              // items published, items with tiles, tiles loaded
};

// Per-lane state of the MMA thread.
struct MmaLane {
  bool done, pend, pend_first, pend_last, first;
  int pend_item, pend_T;
  int tiles_left;
  int I, Iq, Ipv, T;         // items seen, items whose first S / first P V was issued, tiles
};

template <int D, bool BF16, bool TRACE>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Sm100Params P) {
  using namespace ptx;
  constexpr int PANELS = D / 64;
  constexpr uint32_t Q_BYTES = 128u * D * 2u;
  const Problem& p = P.p;

  using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  OutT* const o_base = static_cast<OutT*>(P.o);
  if (P.ws.status[0] != HBSA_STATUS_OK) {
    zero_fill_output(o_base, P.o_s0, P.o_s1, 1ll, P.total_q, p.nhead_q, D, P.lse);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* const smem = smem_raw + pad;
  const uint32_t sQ = raw_addr + pad;                 // 2 lanes
  const uint32_t sRing = sQ + 2u * Q_BYTES;           // n_slots slots
  Control* const ctl = reinterpret_cast<Control*>(smem + 2u * Q_BYTES + (uint32_t)P.n_slots * P.slot_bytes);
  const uint32_t bar_ring_full = smem_u32(&ctl->ring_full[0]), bar_ring_empty = smem_u32(&ctl->ring_empty[0]);
  const uint32_t bar_item_full = smem_u32(&ctl->item_full[0][0]), bar_item_done = smem_u32(&ctl->item_done[0][0]);
  const uint32_t bar_q_full = smem_u32(&ctl->q_full[0]), bar_q_free = smem_u32(&ctl->q_free[0]);
  const uint32_t bar_s_full = smem_u32(&ctl->s_full[0]), bar_p_full = smem_u32(&ctl->p_full[0][0]);
  const uint32_t bar_pv_done = smem_u32(&ctl->pv_done[0][0][0]), bar_o_free = smem_u32(&ctl->o_free[0]);
  const uint32_t bar_drain = smem_u32(&ctl->drain);
  volatile int* const abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int i = 0; i < kMaxSlots; ++i) {
      mbar_init(bar_ring_full + 8 * i, 1);
      mbar_init(bar_ring_empty + 8 * i, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_item_full + 8 * i, 1);
      mbar_init(bar_item_done + 8 * i, kLaneWarps + 1);         // softmax warps of the lane + the MMA thread
      mbar_init(bar_p_full + 8 * i, kLaneWarps);
    }
    for (int i = 0; i < 8; ++i) mbar_init(bar_pv_done + 8 * i, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_q_free + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_o_free + 8 * i, kLaneWarps);
    }
    mbar_init(bar_drain, 1);
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
  const int nt0 = P.nt < kSubCols ? P.nt : kSubCols;       // columns of the first / second half of a tile
  const int nt1 = P.nt - nt0;

  if (warp == kProducerWarp) {
    // =============================== work fetch + TMA producer ===============================
    // Walks the same fixed order as the MMA thread: lanes alternate; a turn of a lane loads V of the tile
    // whose K went out at the lane's previous turn, then K of the lane's next tile (fetching the next work
    // item first when the current one has no tile left).
    const ItemRecord* const records = reinterpret_cast<const ItemRecord*>(P.ws.items);
    unsigned long long* const cursor = reinterpret_cast<unsigned long long*>(P.ws.cursor);
    ProdLane st[2];
#pragma unroll
    for (int L = 0; L < 2; ++L) {
      st[L].done = false; st[L].pend_v = false; st[L].pend_tok = 0; st[L].hk = 0; st[L].tiles_left = 0;
      st[L].mrow = p.mask; st[L].cidx = p.csr_idx; st[L].n_reach = 0; st[L].k_begin = 0; st[L].k_len = 0; st[L].kb0 = 0;
      st[L].n_src = 0; st[L].base = 0; st[L].bal = 0u; st[L].bit_next = false; st[L].val_cur = 0; st[L].val_next = 0;
      st[L].blk = -1; st[L].sub = 0; st[L].I = 0; st[L].Iq = 0; st[L].T = 0;
    }
    RingPos rp = {0, 0u};
    Tracer<TRACE> tr;
    tr.init(P.trace, 3, lane == 0);
    const bool csr = p.csr_ptr != nullptr;
    bool ok = P.debug_stall == 0;
    // Two claims ahead: the record of the candidate item is on its way while the current items run, and the
    // atomic of the one after it is in flight.
    long long cand_idx = 0, next_idx = 0;
    if (lane == 0) {
      cand_idx = (long long)atomicAdd(cursor, 1ull);
      next_idx = (long long)atomicAdd(cursor, 1ull);
    }
    cand_idx = __shfl_sync(0xffffffffu, cand_idx, 0);
    next_idx = __shfl_sync(0xffffffffu, next_idx, 0);
    ItemRecord cand_rec = {};
    if (cand_idx < P.total_items) cand_rec = records[cand_idx / P.items_per_row];
    // The first 32 mask entries of the candidate's row are requested one turn after its record, so that neither load
    // is waited for when a lane takes the candidate.
    bool cand_bits_req = false, cand_bit = false;
    int cand_val = 0;
    auto request_cand_bits = [&]() {
      if (csr) {
        cand_val = lane < cand_rec.count ? p.csr_idx[cand_rec.csr_begin + lane] - cand_rec.kb0 : 0;
      } else {
        const uint8_t* mrow = p.mask + cand_rec.hk * p.mask_s0 + cand_rec.qb * p.mask_s1 + (long long)cand_rec.kb0 * p.mask_s2;
        cand_bit = lane < cand_rec.n_reach && mrow[(long long)lane * p.mask_s2] != 0;
      }
      cand_bits_req = true;
    };

    auto acquire = [&]() -> bool {                       // the ring slot at rp is free again
      return warp_wait(bar_ring_empty + 8u * (uint32_t)rp.slot, rp.phase ^ 1u, abort_flag, budget);
    };

    auto turn = [&](ProdLane& s, const int L) {
      if (!cand_bits_req && cand_idx < P.total_items) request_cand_bits();
      if (s.pend_v) {
        if (!acquire()) { ok = false; return; }
        if (lane == 0) {
          const uint32_t bar = bar_ring_full + 8u * (uint32_t)rp.slot;
          const uint32_t dst = sRing + (uint32_t)rp.slot * P.slot_bytes;
          mbar_arrive_expect_tx(bar, kv_tile_bytes);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(dst + pn * kv_panel_bytes, &tm_v, bar, pn * 64, s.hk, s.pend_tok);
        }
        rp.advance(P.n_slots);
        s.pend_v = false;
        tr.put(0x10 + L);
      }
      if (s.done) return;
      while (s.tiles_left == 0) {
        // ---- next work item of this lane
        const long long idx = cand_idx;
        const bool have = idx < P.total_items;
        if (have && !cand_bits_req) request_cand_bits();
        const ItemRecord rec = cand_rec;
        const bool rec_bit = cand_bit;
        const int rec_val = cand_val;
        const int rem = have ? (int)(idx % P.items_per_row) : 0;
        cand_idx = next_idx;
        cand_bits_req = false;
        if (have) {
          if (cand_idx < P.total_items) cand_rec = records[cand_idx / P.items_per_row];
          if (lane == 0) next_idx = (long long)atomicAdd(cursor, 1ull);
          next_idx = __shfl_sync(0xffffffffu, next_idx, 0);
        }
        const int hsub = rem / P.tiles_per_qblock, qt = rem % P.tiles_per_qblock;
        const int tile_tok0 = rec.q_begin + qt * P.tt;
        if (have && tile_tok0 >= rec.q_end) continue;          // M tile past the ragged end of the q-block
        const int head0 = rec.hk * p.group + hsub * P.gp;
        const int n_tiles = have ? rec.n_tiles : -1;
        // publish: slot I & 1 of the lane is free once every consumer has left item I - 2
        if (s.I >= 2 && !warp_wait(bar2(bar_item_done + 16u * L, s.I), par2(s.I - 2), abort_flag, budget)) { ok = false; return; }
        if (lane == 0) {
          volatile ItemSlot* sl = &ctl->slot[L][s.I & 1];
          sl->n_tiles = n_tiles;
          sl->tile_tok0 = tile_tok0;
          sl->head0 = head0;
          sl->q_end = rec.q_end;
          sl->qi0 = rec.q_in0 + qt * P.tt;
          sl->k_len = rec.k_len;
          sl->off = rec.off;
          __threadfence_block();
          mbar_arrive(bar2(bar_item_full + 16u * L, s.I));
        }
        ++s.I;
        tr.put(0x20 + L);
        if (!have) { s.done = true; return; }
        if (n_tiles <= 0) continue;
        // Q of the lane has one buffer: the last S of the lane's previous item must be done
        if (s.Iq >= 1 && !warp_wait(bar_q_free + 8u * L, (uint32_t)(s.Iq - 1) & 1u, abort_flag, budget)) { ok = false; return; }
        if (lane == 0) {
          const uint32_t bar = bar_q_full + 8u * L;
          mbar_arrive_expect_tx(bar, Q_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_3d(sQ + (uint32_t)L * Q_BYTES + pn * (128u * 128u), &tm_q, bar, pn * 64, head0, tile_tok0);
        }
        ++s.Iq;
        tr.put(0x30 + L);
        s.hk = rec.hk;
        s.tiles_left = n_tiles;
        s.n_reach = rec.n_reach;
        s.k_begin = rec.k_begin;
        s.k_len = rec.k_len;
        s.kb0 = rec.kb0;
        s.base = -32;
        s.bal = 0u;
        s.blk = -1;
        s.sub = 0;
        if (csr) {
          s.cidx = p.csr_idx + rec.csr_begin;
          s.n_src = rec.count;
          s.val_next = rec_val;
        } else {
          s.mrow = p.mask + rec.hk * p.mask_s0 + rec.qb * p.mask_s1 + (long long)rec.kb0 * p.mask_s2;
          s.n_src = rec.n_reach;
          s.bit_next = rec_bit;
        }
      }
      // ---- first row (in-sample) of the lane's next active K/V tile
      int k0 = -1;
      while (true) {
        if (s.blk >= 0 && s.sub < P.n_sub) {
          k0 = s.blk * p.kbs + s.sub * P.nt;
          if (k0 < s.k_len) { ++s.sub; break; }
        }
        while (s.bal == 0u) {                                  // next chunk of 32 entries; they were requested a chunk ago
          s.base += 32;
          const int jn = s.base + 32 + lane;
          if (csr) {
            const int n = s.n_src - s.base;
            s.bal = n >= 32 ? 0xffffffffu : (n > 0 ? (1u << n) - 1u : 0u);
            s.val_cur = s.val_next;
            s.val_next = jn < s.n_src ? s.cidx[jn] - s.kb0 : 0;
          } else {
            s.bal = __ballot_sync(0xffffffffu, s.bit_next);
            s.bit_next = jn < s.n_src && s.mrow[(long long)jn * p.mask_s2] != 0;
          }
          if (s.base >= s.n_src) { s.bal = 0u; break; }         // cannot happen while tiles are left; keeps the loop finite
        }
        if (s.bal == 0u) { ok = false; if (lane == 0) *abort_flag = 1; return; }
        const int pos = __ffs(s.bal) - 1;
        s.bal &= s.bal - 1;
        s.blk = csr ? __shfl_sync(0xffffffffu, s.val_cur, pos) : s.base + pos;
        s.sub = 0;
      }
      if (!acquire()) { ok = false; return; }
      if (lane == 0) {
        ctl->tile_k0[L][s.T & (kTileInfo - 1)] = k0;
        __threadfence_block();
        const uint32_t bar = bar_ring_full + 8u * (uint32_t)rp.slot;
        const uint32_t dst = sRing + (uint32_t)rp.slot * P.slot_bytes;
        mbar_arrive_expect_tx(bar, kv_tile_bytes);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(dst + pn * kv_panel_bytes, &tm_k, bar, pn * 64, s.hk, s.k_begin + k0);
      }
      rp.advance(P.n_slots);
      tr.put(0x40 + L);
      s.pend_v = true;
      s.pend_tok = s.k_begin + k0;
      ++s.T;
      --s.tiles_left;
    };

    while (ok && !(st[0].done && st[1].done && !st[0].pend_v && !st[1].pend_v)) {
      turn(st[0], 0);
      if (!ok) break;
      turn(st[1], 1);
    }
    tr.done();
    // Copies that were issued are always waited for by the MMA thread (it gives up only on barriers
    // of its own sequence), and the CTA does not retire before that thread is through.
  } else if (warp == kMmaWarp) {
    // =============================== MMA issuer ===============================
    // One thread issues every tcgen05.mma of the CTA.  Lanes alternate; a turn of a lane issues P V of the
    // lane's tile in flight (two groups of up to 64 keys, each as soon as its P is there) and then S of the
    // lane's next tile.  S(t+1) goes into the columns P(t) occupies: instructions of one thread execute in
    // issue order, so P V(t) has read P(t) before S(t+1) writes.
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc(BF16, false, false, 128, P.nt);
      const uint32_t idesc_pv = make_idesc(BF16, false, true, 128, D);
      const uint32_t desc_hi = smem_desc_hi(1024u);
      const uint32_t kpanel_units = kv_panel_bytes >> 4;
      const uint32_t slot_units = P.slot_bytes >> 4;
      // Q and K are K-major: 16 head dims further = 32 bytes = 2 descriptor units inside a 64-dim panel.
      // V is MN-major: 16 keys further = 2048 bytes = 128 units.  P: 8 TMEM columns per 16 keys.
      uint64_t qd[2][D / 16];
      uint32_t koff[D / 16];
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t qo = (uint32_t)(ks >> 2) * 1024u + (uint32_t)(ks & 3) * 2u;
        qd[0][ks] = smem_desc_join(smem_desc_lo(sQ, 16u) + qo, desc_hi);
        qd[1][ks] = smem_desc_join(smem_desc_lo(sQ + Q_BYTES, 16u) + qo, desc_hi);
        koff[ks] = (uint32_t)(ks >> 2) * kpanel_units + (uint32_t)(ks & 3) * 2u;
      }
      const uint32_t k_lo0 = smem_desc_lo(sRing, 16u);
      const uint32_t v_lo0 = smem_desc_lo(sRing, kv_panel_bytes);
      const int ks0 = nt0 >> 4, ks1 = nt1 >> 4;
      MmaLane ml[2];
#pragma unroll
      for (int L = 0; L < 2; ++L) {
        ml[L].done = false; ml[L].pend = false; ml[L].pend_first = false; ml[L].pend_last = false; ml[L].first = false;
        ml[L].pend_item = 0; ml[L].pend_T = 0; ml[L].tiles_left = 0;
        ml[L].I = 0; ml[L].Iq = 0; ml[L].Ipv = 0; ml[L].T = 0;
      }
      RingPos rc = {0, 0u};
      Tracer<TRACE> tr;
      tr.init(P.trace, 0, true);
      bool ok = true;
      auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
        const bool r = mbar_wait_bounded(bar, parity, abort_flag, budget);
#ifdef HBSA_STRICT_TCGEN05
        tc_fence_after();
#endif
        return r;
      };

      auto turn = [&](MmaLane& s, const int L) {
        const uint32_t tS = tmem_base + (uint32_t)L * kTmemSStride;
        const uint32_t tO = tmem_base + kTmemOBase + (uint32_t)L * D;
        if (s.pend) {
          // ---- O (+)= P V of the lane's tile in flight; its V tile is the next ring entry
          tr.put(0x10 + L);
          if (!wait(bar_ring_full + 8u * (uint32_t)rc.slot, rc.phase)) { ok = false; return; }
          tr.put(0x20 + L);
          // the first P V of an item overwrites O: the epilogue of the lane's previous item must have read it
          if (s.pend_first && s.Ipv >= 1 && !wait(bar_o_free + 8u * L, (uint32_t)(s.Ipv - 1) & 1u)) { ok = false; return; }
          const uint32_t v_lo = v_lo0 + (uint32_t)rc.slot * slot_units;
          const uint32_t par = (uint32_t)s.pend_T & 1u;
          if (!wait(bar_p_full + 16u * L, par)) { ok = false; return; }
          tr.put(0x30 + L);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            if (ks < ks0) mma_ts(tO, tS + (uint32_t)ks * 8u, smem_desc_join(v_lo + (uint32_t)ks * 128u, desc_hi), idesc_pv,
                                 (s.pend_first && ks == 0) ? 0u : 1u);
          tc_commit(pv_bar(bar_pv_done, L, 0, s.pend_T));
          tr.put(0x40 + L);
          if (ks1 > 0) {
            if (!wait(bar_p_full + 16u * L + 8u, par)) { ok = false; return; }
            tr.put(0x50 + L);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              if (ks < ks1) mma_ts(tO, tS + 32u + (uint32_t)ks * 8u, smem_desc_join(v_lo + (uint32_t)(4 + ks) * 128u, desc_hi), idesc_pv, 1u);
            tc_commit(pv_bar(bar_pv_done, L, 1, s.pend_T));
          }
          tc_commit(bar_ring_empty + 8u * (uint32_t)rc.slot);
          tr.put(0x60 + L);
          rc.advance(P.n_slots);
          if (s.pend_first) ++s.Ipv;
          if (s.pend_last) mbar_arrive(bar2(bar_item_done + 16u * L, s.pend_item));   // through with the item
          s.pend = false;
        }
        if (s.done) return;
        while (s.tiles_left == 0) {
          if (!wait(bar2(bar_item_full + 16u * L, s.I), par2(s.I))) { ok = false; return; }
          const int n_tiles = ctl->slot[L][s.I & 1].n_tiles;
          if (n_tiles < 0) { s.done = true; return; }
          if (n_tiles == 0) {
            mbar_arrive(bar2(bar_item_done + 16u * L, s.I));
            ++s.I;
            continue;
          }
          s.tiles_left = n_tiles;
          s.first = true;
        }
        // ---- S = Q K^T of the lane's next tile; its K tile is the next ring entry
        tr.put(0x70 + L);
        if (!wait(bar_ring_full + 8u * (uint32_t)rc.slot, rc.phase)) { ok = false; return; }
        tr.put(0x80 + L);
        if (s.first && !wait(bar_q_full + 8u * L, (uint32_t)s.Iq & 1u)) { ok = false; return; }
        tr.put(0x90 + L);
#ifdef HBSA_STRICT_TCGEN05
        // every P V group of the lane has completed before S overwrites the columns of P
        if (s.T >= 1 && !wait(pv_bar(bar_pv_done, L, ks1 > 0 ? 1 : 0, s.T - 1), pv_par(s.T - 1))) { ok = false; return; }
#endif
        const uint32_t k_lo = k_lo0 + (uint32_t)rc.slot * slot_units;
        if (L == 0) {
          mma_ss_c<false>(tS, qd[0][0], smem_desc_join(k_lo + koff[0], desc_hi), idesc_qk);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) mma_ss_c<true>(tS, qd[0][ks], smem_desc_join(k_lo + koff[ks], desc_hi), idesc_qk);
        } else {
          mma_ss_c<false>(tS, qd[1][0], smem_desc_join(k_lo + koff[0], desc_hi), idesc_qk);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) mma_ss_c<true>(tS, qd[1][ks], smem_desc_join(k_lo + koff[ks], desc_hi), idesc_qk);
        }
        tc_commit(bar_s_full + 8u * L);
        tc_commit(bar_ring_empty + 8u * (uint32_t)rc.slot);
        if (s.tiles_left == 1) tc_commit(bar_q_free + 8u * L);             // the lane's Q buffer may be refilled
        tr.put(0xa0 + L);
        rc.advance(P.n_slots);
        s.pend = true;
        s.pend_first = s.first;
        s.pend_last = s.tiles_left == 1;
        s.pend_item = s.I;
        s.pend_T = s.T;
        ++s.T;
        if (s.first) { ++s.Iq; s.first = false; }
        if (--s.tiles_left == 0) ++s.I;
      };

      while (ok && !(ml[0].done && ml[1].done && !ml[0].pend && !ml[1].pend)) {
        turn(ml[0], 0);
        if (!ok) break;
        turn(ml[1], 1);
      }
      tr.done();
      // Every product issued so far has completed before the CTA gives TMEM back (bounded).
      tc_commit(bar_drain);
      mbar_wait_bounded(bar_drain, 0u, abort_flag, budget);
    }
    __syncwarp();
  } else {
    // =============================== softmax + epilogue ===============================
    const int L = warp >> 2, wq = warp & 3;
    const int row = wq * 32 + lane;                  // 0..127: row of the M tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
    const uint32_t tSlane = tmem_base + (uint32_t)L * kTmemSStride + lane_off;
    const uint32_t tOmine = tmem_base + kTmemOBase + (uint32_t)L * D + lane_off;
    const float scale_log2 = P.scale_log2;
    const int n_half = nt1 > 0 ? 2 : 1;
    Tracer<TRACE> tr;
    tr.init(P.trace, 1 + L, wq == 0 && lane == 0);
    int I = 0, T = 0;
    bool ok = true;
    while (ok) {
      ok = warp_wait(bar2(bar_item_full + 16u * L, I), par2(I), abort_flag, budget);
      if (!ok) break;
      const volatile ItemSlot* sl = &ctl->slot[L][I & 1];
      const int n_tiles = sl->n_tiles;
      if (n_tiles < 0) break;
      tr.put(0x10);
      const int tile_tok0 = sl->tile_tok0, head0 = sl->head0, q_end = sl->q_end;
      const int r_tok = tile_tok0 + (row >> P.gp_shift), r_head = head0 + (row & (P.gp - 1));
      if (n_tiles == 0) {
        // No active k-block: the rows are exact zeros (fwd_triton_fix_tile_size.py:189).
        if (r_tok < q_end) {
          uint4* dst = reinterpret_cast<uint4*>(o_base + r_tok * P.o_s0 + r_head * P.o_s1);
#pragma unroll
          for (int i = 0; i < D / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
          if (P.lse != nullptr) P.lse[(long long)r_tok * p.nhead_q + r_head] = -INFINITY;
        }
      } else {
        int limit_row = sl->k_len - 1;
        if (p.causal) limit_row = min(limit_row, sl->qi0 + (row >> P.gp_shift) + sl->off);
        float m_ref = -INFINITY, l = 0.f;
        for (int t = 0; t < n_tiles && ok; ++t, ++T) {
          ok = warp_wait(bar_s_full + 8u * L, (uint32_t)T & 1u, abort_flag, budget);
          if (!ok) break;
          tc_fence_after();
          tr.put(0x20);
          const int tile_col0 = ctl->tile_k0[L][T & (kTileInfo - 1)];
          for (int h = 0; h < n_half && ok; ++h) {
            const int my_nc = h == 0 ? nt0 : nt1;                          // columns of this half: 16, 32, 48 or 64
            const int col_limit = limit_row - tile_col0 - h * kSubCols;    // columns <= col_limit are valid
            const uint32_t tSmine = tSlane + (uint32_t)h * kSubCols;       // S of this half
            const uint32_t tPmine = tSlane + (uint32_t)h * (kSubCols / 2); // P of this half (16-bit pairs)
            // on the causal diagonal or at the ragged end of the sample; decided per warp, because the two code paths
            // below both contain warp-wide TMEM stores (rows that are not on the edge mask nothing)
            const bool edge = __any_sync(0xffffffffu, col_limit < my_nc - 1);
            // ---- this thread's row of S of this half, all in registers before its first P is stored (P of the second
            //      half lands on S columns of the first half, which are in registers by then).  Load and wait stay in
            //      one straight piece of code: the registers of an asynchronous TMEM load must not be moved by the
            //      compiler before the wait.
            uint32_t r[64];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (my_nc > 16 * j) tmem_ld16(tSmine + 16 * j, *reinterpret_cast<uint32_t(*)[16]>(&r[16 * j]));
            tmem_wait_ld();
            if (h == 0) tr.put(0x21);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pmax0 = 0u, pmax1 = 0u;
            bool exact = t == 0 && h == 0;                 // first columns of the item: the maximum must come first
            if (!exact) {
              // Optimistic pass: exponentials against the reference maximum of the previous columns (any
              // reference gives the same softmax; it only has to keep P in range).  If a P turns out to
              // exceed 2^8, the exact pass below redoes these columns.
              const float neg_m0 = m_ref == -INFINITY ? 0.f : -m_ref;
              if (edge) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (my_nc > 16 * j) {
#pragma unroll
                    for (int i = 16 * j; i < 16 * j + 16; ++i)
                      if (i > col_limit) r[i] = 0xff800000u;                 // -inf: exp2 makes it an exact 0
                    uint32_t pk[8];
                    exp16<BF16, 0>(&r[16 * j], pk, scale_log2, neg_m0, sum);
                    tmem_st8(tPmine + 8 * j, pk);
                    pmax0 = __vimax3_u16x2(pmax0, pk[0], pk[1]);
                    pmax1 = __vimax3_u16x2(pmax1, pk[2], pk[3]);
                    pmax0 = __vimax3_u16x2(pmax0, pk[4], pk[5]);
                    pmax1 = __vimax3_u16x2(pmax1, pk[6], pk[7]);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (my_nc > 16 * j) {
                    uint32_t pk[8];
                    exp16<BF16, HBSA_POLY_PAIRS>(&r[16 * j], pk, scale_log2, neg_m0, sum);
                    tmem_st8(tPmine + 8 * j, pk);
                    // P >= 0: 16-bit floats order like unsigned integers, two per word, three words per instruction
                    pmax0 = __vimax3_u16x2(pmax0, pk[0], pk[1]);
                    pmax1 = __vimax3_u16x2(pmax1, pk[2], pk[3]);
                    pmax0 = __vimax3_u16x2(pmax0, pk[4], pk[5]);
                    pmax1 = __vimax3_u16x2(pmax1, pk[6], pk[7]);
                  }
                }
              }
              tr.put(0x22);
              // A P above 2^8 means the columns exceed the reference by more than the threshold; the row maximum
              // itself is only computed on that (rare) path.  Rows without a reference yet take it as well.
              const uint32_t pm = __vimax3_u16x2(pmax0, pmax1, 0u);
              const uint32_t p_hi = max(pm >> 16, pm & 0xffffu);
              bool need = p_hi > (BF16 ? 0x4380u : 0x5c00u) || m_ref == -INFINITY;
              if (__any_sync(0xffffffffu, need)) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (my_nc > 16 * j) max16(&r[16 * j], mx4);
                const float mx_s = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale > 0 keeps the order
                need = mx_s > m_ref + kRescaleThreshold;
                if (__any_sync(0xffffffffu, need)) {       // (a row without reference whose columns are all masked needs nothing)
                  // O and l move to the new reference maximum; needs the previous P V group of the lane
                  const int hp = h == 1 ? 0 : n_half - 1, Tp = h == 1 ? T : T - 1;
                  ok = warp_wait(pv_bar(bar_pv_done, L, hp, Tp), pv_par(Tp), abort_flag, budget);
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
                  exact = true;                            // P of these columns is recomputed against the new reference
                  sum[0] = sum[1] = sum[2] = sum[3] = 0.f;
                }
              }
            } else {
              if (edge) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                  if (i > col_limit) r[i] = 0xff800000u;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (my_nc > 16 * j) max16(&r[16 * j], mx4);
              m_ref = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            }
            if (exact) {
              // ---- P = exp2(S * scale - m) packed to 16 bit, row sum
              const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (my_nc > 16 * j) {
                  uint32_t pk[8];
                  exp16<BF16, 0>(&r[16 * j], pk, scale_log2, neg_m, sum);
                  tmem_st8(tPmine + 8 * j, pk);
                }
              }
            }
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tr.put(0x23);
            tmem_wait_st();
            tr.put(0x24);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full + 16u * L + 8u * (uint32_t)h);   // one arrival per warp
            tr.put(0x30 + h);
          }
        }
        if (!ok) break;

        // ---- epilogue: O / l -> global; rows past the q-block end are dropped, rows that saw no key are zeros
        const bool live = l > 0.f;
        const float inv = live ? 1.f / l : 0.f;
        const uint64_t inv2 = pack_f32x2(inv, inv);
        const bool store_row = r_tok < q_end;
        if (P.lse != nullptr && store_row) {
          // ln sum exp of the row's scaled scores = ln 2 * (reference + log2 l), whatever reference was used
          P.lse[(long long)r_tok * p.nhead_q + r_head] = live ? 0.6931471805599453f * (m_ref + log2f(l)) : -INFINITY;
        }
        tr.put(0x40);
        ok = warp_wait(pv_bar(bar_pv_done, L, n_half - 1, T - 1), pv_par(T - 1), abort_flag, budget);
        if (!ok) break;
        tc_fence_after();
        tr.put(0x50);
        OutT* const orow = o_base + r_tok * P.o_s0 + r_head * P.o_s1;
        // 64 columns of O per TMEM round trip (128 would not fit the registers of a thread beside the packing)
#pragma unroll
        for (int cb = 0; cb < D; cb += 64) {
          uint32_t oa[64];
          tmem_ld32(tOmine + cb, *reinterpret_cast<uint32_t(*)[32]>(&oa[0]));
          tmem_ld32(tOmine + cb + 32, *reinterpret_cast<uint32_t(*)[32]>(&oa[32]));
          tmem_wait_ld();
          if (cb + 64 >= D) {
            tc_fence_before();                                             // O is in registers: the lane's next item may overwrite it
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_o_free + 8u * L);
          }
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float y0, y1;
              unpack_f32x2(mul_f32x2(pack_b32x2(oa[c0 + e], oa[c0 + e + 1]), inv2), y0, y1);
              w[e >> 1] = live ? pack2<BF16>(y0, y1) : 0u;
            }
            if (store_row) {
              // this thread's 64 bytes of the row: two 256-bit stores when the rows are 32-byte aligned
              if (P.o_vec32) {
                st_global_v8(orow + cb + c0, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
                st_global_v8(orow + cb + c0 + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  *reinterpret_cast<uint4*>(orow + cb + c0 + 8 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
              }
            }
          }
        }
        tr.put(0x60);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar2(bar_item_done + 16u * L, I));
      ++I;
    }
    tr.done();
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

long long* g_trace = nullptr;
long long g_wait_budget = 4000000000ll;   // clock64 ticks a wait inside the kernel may take (about two seconds)
int g_debug_stall = 0;

}  // namespace

void sm100_set_wait_budget(long long clocks, int stall_producer) {
  g_wait_budget = clocks > 0 ? clocks : 4000000000ll;
  g_debug_stall = stall_producer ? 1 : 0;
}

void sm100_set_trace(long long* device_buffer) { g_trace = device_buffer; }
size_t sm100_trace_bytes() { return (size_t)kTraceRegions * kTraceCap * sizeof(long long); }

int sm100_kv_tile_rows(int kbs) {
  if (kbs <= kTileRowsMax) return kbs;
  for (int nt = kTileRowsMax; nt >= 16; nt -= 16)
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
  P.debug_stall = g_debug_stall;
  P.trace = g_trace;
  P.o_vec32 = ((uintptr_t)a.o % 32 == 0 && (a.o_stride[0] * 2) % 32 == 0 && (a.o_stride[1] * 2) % 32 == 0) ? 1 : 0;

  P.total_items = (long long)p.nhead_k * p.num_q_block * P.items_per_row;
  if (P.total_items <= 0) { *err_text = "no work items"; return HBSA_ERR_SHAPE; }
  const long long pairs = (P.total_items + 1) / 2;               // two items in flight per persistent CTA
  const long long resident = sm_count();
  const unsigned grid = (unsigned)(pairs < resident ? pairs : resident);

  // shared memory: two Q tiles, the K/V ring, the control block, and up to 1023 bytes of alignment slack
  const size_t q_bytes = 2u * 128u * (size_t)p.headdim * 2u;
  P.slot_bytes = (uint32_t)P.nt * (uint32_t)p.headdim * 2u;       // a multiple of 1024 for every legal (nt, headdim)
  const size_t fixed = q_bytes + sizeof(Control) + 1024u;
  long long n_slots = ((long long)kSmemLimit - (long long)fixed) / (long long)P.slot_bytes;
  if (n_slots > kMaxSlots) n_slots = kMaxSlots;
  if (n_slots < kMinSlots) { *err_text = "shared memory cannot hold the K/V ring"; return HBSA_ERR_UNSUPPORTED; }
  P.n_slots = (int)n_slots;
  size_t smem = fixed + (size_t)P.n_slots * P.slot_bytes;
  if (smem < kSmemLimit / 2 + 1024) smem = kSmemLimit / 2 + 1024;  // one CTA per SM: each one takes all 512 TMEM columns

  CUtensorMap tq, tk, tv;
  if (!encode_map(fn, &tq, bf16, a.q, p.headdim, p.nhead_q, a.total_q, a.q_stride[0], a.q_stride[1], gp, P.tt) ||
      !encode_map(fn, &tk, bf16, a.k, p.headdim, p.nhead_k, a.total_k, a.k_stride[0], a.k_stride[1], 1, P.nt) ||
      !encode_map(fn, &tv, bf16, a.v, p.headdim, p.nhead_k, a.total_k, a.v_stride[0], a.v_stride[1], 1, P.nt)) {
    *err_text = "cuTensorMapEncodeTiled rejected a q/k/v layout";
    return HBSA_ERR_UNSUPPORTED;
  }

  cudaError_t e = cudaSuccess;
#define HBSA_LAUNCH_SM100(D_, BF_, TR_)                                                                   \
  do {                                                                                                   \
    e = cudaFuncSetAttribute(fwd_sm100_kernel<D_, BF_, TR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) {                                                                              \
      fwd_sm100_kernel<D_, BF_, TR_><<<grid, kThreads, smem, stream>>>(tq, tk, tv, P);                   \
      e = cudaGetLastError();                                                                            \
    }                                                                                                    \
  } while (0)
#define HBSA_LAUNCH_SM100_T(D_, BF_) do { if (P.trace != nullptr) HBSA_LAUNCH_SM100(D_, BF_, true); else HBSA_LAUNCH_SM100(D_, BF_, false); } while (0)
  if (p.headdim == 128) { if (bf16) HBSA_LAUNCH_SM100_T(128, true); else HBSA_LAUNCH_SM100_T(128, false); }
  else { if (bf16) HBSA_LAUNCH_SM100_T(64, true); else HBSA_LAUNCH_SM100_T(64, false); }
#undef HBSA_LAUNCH_SM100_T
#undef HBSA_LAUNCH_SM100
  if (e != cudaSuccess) { *err_text = cudaGetErrorString(e); return (int)e; }
  return 0;
}

}  // namespace hbsa
