// Score form on the tcgen05 tensor cores, bf16, head dimension 64: one CTA owns ONE
// 128-row tile and walks column tiles that alternate between two groups of compute warps
// ("ping-pong"), each with its own S / W / E / P regions in TMEM.
//
//   MODE_DQ    grad_q:  rows = queries (x = q, u = gs), columns = keys (y = k, z = v)
//              E = f'(x.y) (u.z - dvec_row);          grad_q += E Y
//   MODE_DKDV  grad_k and grad_v in one pass: rows = keys (x = k, u = v), columns =
//              queries (y = q, z = gs), reverse direction (column >= row - off)
//              E = f'(x.y) (u.z - dvec_col), P = f(x.y);  grad_k += E Y,  grad_v += P Z
//   MODE_FWD   forward: rows = queries (x = q), columns = keys (y = k, z = v)
//              P = f(x.y);  O += P Z,  den = row sums of P,  out = O / den
// The gradients use 64-column tiles (S and W double-buffered fill TMEM); the forward has no
// W and uses 128-column tiles, which halves the barrier hand-offs per score.
//
// Why this shape.  Per column tile the chain is S-MMA -> TMEM load -> polynomial on the CUDA
// cores -> TMEM store -> accumulating MMA, and the round trip between the tensor pipe and the
// CUDA cores (commit, barrier, tcgen05.ld latency) is as long as the MMAs themselves.  Two
// groups working on alternate tiles keep two such chains in flight on the same rows, sixteen
// compute warps (four per scheduler) hide the TMEM and FP32 latencies inside a chain, and
// grad_k / grad_v share S, so a tile costs four products instead of five.
//
// TMEM columns: S[2] 0..127 | W[2] 128..255 | E[2] 256..319 (bf16 pairs) | P[2] 320..383 |
// accumulator 384..447 | second accumulator 448..511.  Forward: three sets of 128 score columns at 0, 128,
// 256 (tile j in set j % 3, group j % 2), P written over the S columns it came from, accumulator 384..447.
// Warps 0-7 are group 0 (even tiles), 8-15 group 1 (odd tiles); inside a group warp % 4 is
// the TMEM lane quarter (32 rows) and (warp / 4) % 2 picks one half of the tile's columns.  Warp 16 is
// the TMA producer, warps 17 and 18 issue the S / W products of group 0 and group 1 (warp 17
// also allocates TMEM; in the forward it issues every S product, in tile order, and warp 18 idles),
// warp 19 issues the accumulating products.
// All waits are bounded; a wait that gives up records a status and the CTA winds down.
#include <climits>
#include <cstdlib>
#include <type_traits>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_wtc_status = 0;

namespace {
using namespace sm100;

struct WArgs {
  void* o;               // (heads, nrows, 64) bf16: out, grad_q, or grad_k
  void* o2;              // MODE_DKDV: grad_v
  float* den_out;        // MODE_FWD: (heads, nrows) row sums
  const float* den_add;  // MODE_FWD: added to the row sum (may be null)
  const float* o_add;    // fp32 rows added before rounding (may be null)
  const float* o2_add;
  const void* x;         // row operand in global memory (normalisation dots)
  const float* dvec;     // (heads, nq)
  float* dots;           // per head sum of o . x, or null
  const stat_t* stat_q;
  const stat_t* stat_k;
  int nrows, ncols, off, mask, ntr, chunk;
  float a0, a1, a2, lim;
  int o_heads;           // MODE_FWD: > 0 writes out as (batch, nrows, o_heads, 64)
};

enum { MODE_DQ = 0, MODE_DKDV = 1, MODE_FWD = 2 };
constexpr int BM = 128, D = 64;
constexpr int kThreads = 640;
constexpr int kProducerWarp = 16, kIssuerWarp = 17, kAccIssuerWarp = 19, kComputeWarps = 16;  // warps 17, 18: S / W issuers
constexpr int ROW_TILE = BM * 128;
constexpr int OFF_X = 0, OFF_U = ROW_TILE;
constexpr int T_S = 0, T_W = 128, T_E = 256, T_P = 320, T_O = 384, T_O2 = 448;
constexpr int T_X = T_P;   // MODE_DQ (no P): the row operands x (32 columns) and u (32 columns) as TMEM A operands
// Forward: three sets of 128 score columns (tile j in set j % 3) at 0, 128, 256; P overwrites the S columns its
// warp has just read (16 packed columns at the start of every 32), so no separate P region is needed.
constexpr int kSets = 3, SET_COLS = 128;
template <int MODE>
struct WCfg {
  static constexpr int BN = (MODE == MODE_FWD) ? 128 : 64;   // columns per tile
  // Ring stages of (Y tile, Z tile).  The count must be even: the two S / W issuer warps take
  // alternate tiles, and with an even count each stage barrier is only ever waited on by one of
  // them, on consecutive phases.  With an odd count a stage alternates between the two warps, each
  // would wait on every second phase of its barrier -- always the same parity -- and a parity wait
  // cannot tell "the phase before mine has not completed yet" from "mine has completed": when the
  // loads arrive late and out of order (many heads streaming from DRAM at once) the warp then issues
  // on a stage that is still being written and the CTA can finish with loads in flight.
  static constexpr int NS = (MODE == MODE_FWD) ? 6 : 8;
  static_assert(NS % 2 == 0, "each stage barrier must belong to one issuer warp");
  static constexpr int COL_TILE = BN * 128, STAGE = 2 * COL_TILE;
  static constexpr int OFF_ST = (MODE == MODE_FWD ? 1 : 2) * ROW_TILE;   // the forward has no U tile
  static constexpr int OFF_VEC = OFF_ST + NS * STAGE;      // per compute warp 2 x 32 floats
  static constexpr int OFF_BAR = OFF_VEC + kComputeWarps * 2 * 32 * 4;
  static constexpr int NBAR = 2 + 2 * NS + 9;
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_wtc_status, 0, code); }

// GQ: grouped k/v heads (bh > bhkv); the plain case compiles without the head walk.
// SQ (MODE_DKDV without grouped heads, a2 > 0): the polynomial in completed-square form,
//   f(s) = A2 ((s + b)^2 + c),  f'(s) = 2 A2 (s + b),  b = A1 / (2 A2),  c = A0 / A2 - b^2,
// so that a pair of scores costs t = s + b, P' = t t + c, E' = t (w - dvec): four packed operations
// instead of five.  The factors A2 (grad_v) and 2 A2 (grad_k) multiply the accumulators in the epilogue.
template <int MODE, bool GQ, bool SQ = false>
__global__ void __launch_bounds__(kThreads, 1)
dense_tc_wide_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU,
                     const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmZ,
                     const WArgs a, const int kv_ratio) {
  using C = WCfg<MODE>;
  constexpr bool FUSED = MODE == MODE_DKDV, FWD = MODE == MODE_FWD;
  constexpr int BN = C::BN, NS = C::NS, COL_TILE = C::COL_TILE, STAGE = C::STAGE;
  constexpr int OFF_ST = C::OFF_ST, OFF_VEC = C::OFF_VEC, OFF_BAR = C::OFF_BAR, OFF_TMEM = C::OFF_TMEM;
  constexpr bool PV_EARLY = MODE == MODE_DQ;
  // grad_q has 64 TMEM columns to spare: its row operands are copied there once, so that the S / W
  // products read only the column tile from shared memory (32.6 instead of 48.6 cycles per K=16 step)
  constexpr bool XT = MODE == MODE_DQ;
  // Forward: with P written in place a set is 128 columns and three fit beside the accumulator, so a
  // group's next scores are usually waiting when it finishes a tile (with two S buffers released only
  // after the second 32-column pass, the next S product started late).  A set is refilled once the
  // accumulating product of its previous tile is done.  The gradients keep two sets that are released
  // as soon as they are in registers: their E / P need their own columns, and refilling a set only after
  // its accumulating products makes the loop longer than the third set makes it wider (measured:
  // grad_q 18.3 -> 19.5 ms, fused 26.1 -> 29.4 ms, forward 14.3 -> 13.4 ms).
  constexpr bool TRI = FWD;
  constexpr int HB = BN / 2;          // columns of one compute warp = packed bf16 columns of one group
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + OFF_BAR;
  // barrier map: x | done | full[NS] | empty[NS] | s_full[2] | s_free[2] | p_full[2] | pv_done[2]
  const uint32_t BAR_X = bar0, BAR_DONE = bar0 + 8;
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (2 + s); };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (2 + NS + s); };
  auto BAR_S = [&](int g) { return bar0 + 8u * (2 + 2 * NS + g); };
  auto BAR_SFREE = [&](int g) { return bar0 + 8u * (4 + 2 * NS + g); };
  auto BAR_P = [&](int g) { return bar0 + 8u * (6 + 2 * NS + g); };
  auto BAR_PV = [&](int g) { return bar0 + 8u * (8 + 2 * NS + g); };
  const uint32_t BAR_XT = bar0 + 8u * (10 + 2 * NS);
  // TRI reuses the nine words from s_full on: s_full[set] | p_full[set] | set_free[set]
  auto BAR_TS = [&](int t) { return bar0 + 8u * (2 + 2 * NS + t); };
  auto BAR_TP = [&](int t) { return bar0 + 8u * (2 + 2 * NS + kSets + t); };
  auto BAR_TF = [&](int t) { return bar0 + 8u * (2 + 2 * NS + 2 * kSets + t); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool rev = FUSED;
  // consecutive CTAs work on one head (its column tiles stay in L2); longest rows first
  const int head = blockIdx.x / a.ntr;
  const int pidx = blockIdx.x % a.ntr;
  const int rt = rev ? pidx : a.ntr - 1 - pidx;
  const int r0 = rt * BM;

  const int ntile = (a.ncols + BN - 1) / BN;
  int tb = 0, te = ntile;
  if (a.mask) {
    if (rev) tb = max(0, r0 - a.off) / BN;
    else te = min(ntile, (min(r0 + BM - 1, a.nrows - 1) + a.off) / BN + 1);
  }
  if (a.chunk > 0) {  // the row tile lies in one chunk (chunk % 256 == 0)
    const int cb = (r0 / a.chunk) * (a.chunk / BN), ce = cb + a.chunk / BN;
    if (rev) te = min(te, ce);
    else tb = cb;
  }
  // Grouped k/v heads: a query head reads the tiles of key/value head `head / ratio`; a key/value
  // head (MODE_DKDV rows) walks the same tile range once for each of its `ratio` query heads.
  const int ratio = GQ ? kv_ratio : 1;
  const int Jh = max(te - tb, 0);
  const int J = rev ? Jh * ratio : Jh;
  // Column head and tile of the running tile number, advanced without divisions: `t` is the tile
  // inside the head's range [tb, tb + Jh), `h` the column head.
  struct ColPos { int t, h; };
  const ColPos pos0 = {tb, rev ? head * ratio : head / ratio};
  auto advance = [&](ColPos& cp, int steps) {
    if constexpr (GQ) {
      cp.t += steps;
      if (rev)
        while (cp.t >= tb + Jh && Jh > 0) { cp.t -= Jh; ++cp.h; }
    }
  };
  // without grouped heads the position follows from the tile number alone and the tracker is dead code
  auto tile_of = [&](int j, const ColPos& cp) { return GQ ? cp.t : tb + j; };
  auto head_of = [&](const ColPos& cp) { return GQ ? cp.h : head; };

  if (tid == 0) {
    mbar_init(BAR_X, 1);
    mbar_init(BAR_DONE, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR_FULL(s), 1);
      mbar_init(BAR_EMPTY(s), 1);
    }
    if constexpr (TRI) {
      for (int t = 0; t < kSets; ++t) {
        mbar_init(BAR_TS(t), 1);
        mbar_init(BAR_TP(t), kComputeWarps / 2);
        mbar_init(BAR_TF(t), 1);
      }
    } else {
      mbar_init(BAR_XT, kComputeWarps);
      for (int g = 0; g < 2; ++g) {
        mbar_init(BAR_S(g), 1);
        mbar_init(BAR_SFREE(g), kComputeWarps / 2);
        mbar_init(BAR_P(g), kComputeWarps / 2);
        mbar_init(BAR_PV(g), 1);
      }
    }
    mbar_fence_init();
  }
  if (warp == kIssuerWarp) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kProducerWarp) {
    // ================= TMA producer =================
    if (lane == 0 && J > 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmU);
      tma_prefetch_desc(&tmY);
      tma_prefetch_desc(&tmZ);
      mbar_expect_tx(BAR_X, (FWD ? 1 : 2) * ROW_TILE);
      tma_load_3d(sbase + OFF_X, &tmX, BAR_X, 0, r0, head);
      if (!FWD) tma_load_3d(sbase + OFF_U, &tmU, BAR_X, 0, r0, head);
    }
    ColPos pc = pos0;
    for (int j = 0; j < J; ++j, advance(pc, 1)) {
      const int s = j % NS;
      if (!mbar_wait(BAR_EMPTY(s), (((j / NS) & 1) ^ 1))) { report(1); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), STAGE);
        const uint32_t dst = sbase + OFF_ST + s * STAGE;
        tma_load_3d(dst, &tmY, BAR_FULL(s), 0, tile_of(j, pc) * BN, head_of(pc));
        tma_load_3d(dst + COL_TILE, &tmZ, BAR_FULL(s), 0, tile_of(j, pc) * BN, head_of(pc));
      }
    }
  } else if (warp == kIssuerWarp || warp == kIssuerWarp + 1) {
    // ================= MMA issuers of the S / W products, one per group =================
    // The whole warp runs the loop (uniform control flow and operands); one elected lane
    // executes the tcgen05 instructions.  S and W of tile j go to the TMEM regions of group
    // j & 1 as soon as that group has copied tile j - 2 to registers, independently of the
    // accumulating products, which the other issuer warp handles.
    if (TRI && J > 0 && warp == kIssuerWarp) {
      // one warp takes every tile in order (each barrier is waited on phase after phase): S of tile j
      // goes to set j % 3 once the accumulating product of tile j - 3 has read that set's P
      constexpr uint32_t idescS = idesc_bf16(BM, BN, 0, 0);
      const uint32_t x_lo = desc_lo(sbase + OFF_X, 16);
      const uint32_t st_k = desc_lo(sbase + OFF_ST, 16);
      bool ok = mbar_wait_warp(BAR_X, 0);
      if (!ok) report(2);
      tc_fence_after();
      for (int j = 0; ok && j < J; ++j) {
        const int s = j % NS, set = j % kSets;
        if (!mbar_wait_warp(BAR_FULL(s), (uint32_t)((j / NS) & 1))) { report(3); break; }
        if (j >= kSets && !mbar_wait_warp(BAR_TF(set), (uint32_t)(((j / kSets) - 1) & 1))) { report(4); break; }
        tc_fence_after();
        if (elect_one()) {
          umma_ss_k64(tmem + set * SET_COLS, x_lo, st_k + (uint32_t)s * (STAGE >> 4), idescS);
          umma_commit(BAR_TS(set));
        }
        __syncwarp();
      }
    } else if (!TRI && J > 0) {
      constexpr uint32_t idescS = idesc_bf16(BM, BN, 0, 0);
      const uint32_t x_lo = desc_lo(sbase + OFF_X, 16);
      const uint32_t u_lo = desc_lo(sbase + OFF_U, 16);
      const uint32_t st_k = desc_lo(sbase + OFF_ST, 16);         // stage 0, K-major view
      bool ok = mbar_wait_warp(XT ? BAR_XT : BAR_X, 0);
      if (!ok) report(2);
      tc_fence_after();
      const int g = warp - kIssuerWarp;
      for (int j = g; ok && j < J; j += 2) {
        const int s = j % NS;
        // the stage has normally been loaded long ago: checking it first keeps that check out of
        // the s_free -> S ready path, which bounds the group's tile period
        if (!mbar_wait_warp(BAR_FULL(s), (uint32_t)((j / NS) & 1))) { report(3); break; }
        if (j >= 2 && !mbar_wait_warp(BAR_SFREE(g), (uint32_t)(((j >> 1) - 1) & 1))) { report(4); break; }
        tc_fence_after();
        const uint32_t y_lo = st_k + (uint32_t)s * (STAGE >> 4);
        if (elect_one()) {
          if constexpr (XT) {
            umma_ts_k64(tmem + T_S + g * BN, tmem + T_X, y_lo, idescS);
            umma_ts_k64(tmem + T_W + g * BN, tmem + T_X + 32, y_lo + (COL_TILE >> 4), idescS);
          } else {
            umma_ss_k64(tmem + T_S + g * BN, x_lo, y_lo, idescS);
            if (!FWD) umma_ss_k64(tmem + T_W + g * BN, u_lo, y_lo + (COL_TILE >> 4), idescS);
          }
          umma_commit(BAR_S(g));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (warp == kAccIssuerWarp) {
    // ================= MMA issuer of the accumulating products =================
    // The stage of tile j is known to be loaded and S / W of tile j complete once the
    // group's P barrier has fired, so this warp waits on nothing else.
    if (J > 0) {
      constexpr uint32_t idescO = idesc_bf16(BM, D, 0, 1);
      const uint32_t st_mn = desc_lo(sbase + OFF_ST, COL_TILE);  // stage 0, MN-major view
      for (int j = 0; j < J; ++j) {
        const int s = j % NS, g = j & 1;
        const uint32_t y_mn = st_mn + (uint32_t)s * (STAGE >> 4);
        if constexpr (TRI) {
          // P lies where S was: the warp that read columns [32 c, 32 c + 32) of the set left 16 packed
          // columns at 32 c, so K-step ks reads 8 columns at (ks / 2) * 32 + (ks % 2) * 8
          const int set = j % kSets;
          if (!mbar_wait_warp(BAR_TP(set), (uint32_t)((j / kSets) & 1))) { report(5); break; }
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              umma_ts_1(tmem + T_O, tmem + set * SET_COLS + (ks >> 1) * 32 + (ks & 1) * 8,
                        y_mn + (COL_TILE >> 4) + ks * 128, idescO, (j > 0 || ks > 0) ? 1u : 0u);
            umma_commit(BAR_TF(set));
            umma_commit(BAR_EMPTY(s));
            if (j + 1 == J) umma_commit(BAR_DONE);
          }
          __syncwarp();
          continue;
        }
        if (!mbar_wait_warp(BAR_P(g), (uint32_t)((j >> 1) & 1))) { report(5); break; }
        tc_fence_after();
        if (elect_one()) {
          // the gradients multiply E by the Y tile, the forward multiplies P by the Z tile
          umma_ts_steps<BN / 16>(tmem + T_O, tmem + T_E + g * HB, y_mn + (FWD ? (COL_TILE >> 4) : 0), idescO,
                                 j > 0 ? 1u : 0u);
          if (FUSED)
            umma_ts_steps<BN / 16>(tmem + T_O2, tmem + T_P + g * HB, y_mn + (COL_TILE >> 4), idescO,
                                   j > 0 ? 1u : 0u);
          umma_commit(BAR_PV(g));
          umma_commit(BAR_EMPTY(s));
          if (j + 1 == J) umma_commit(BAR_DONE);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ================= compute warps =================
    const int gp = warp >> 3, cpart = (warp >> 2) & 1, qd = warp & 3;
    const int row = r0 + qd * 32 + lane;
    const bool row_ok = row < a.nrows;
    // scale of the scores: query-head statistic times key-head statistic (the query head of a
    // MODE_DKDV tile changes with the tile when k/v heads are grouped)
    const float ck = stat_scale(a.stat_k, rev ? head : head / ratio, a.lim);
    const float c = stat_scale(a.stat_q, rev ? head * ratio : head, a.lim) * stat_scale(a.stat_k, rev ? head : head / ratio, a.lim);
    const float A0 = a.a0, A1 = a.a1 * c, A2 = a.a2 * c * c;
    const uint64_t A0v = pack2(A0, A0);
    using coef_t = typename std::conditional<GQ, uint64_t, const uint64_t>::type;   // fixed unless heads are grouped
    coef_t A1v = pack2(A1, A1), A2v = pack2(A2, A2), A2d = pack2(2.f * A2, 2.f * A2);
    const float sq_b = SQ ? A1 / (2.f * A2) : 0.f, sq_c = SQ ? A0 / A2 - sq_b * sq_b : 0.f;
    const uint64_t Bv = pack2(sq_b, sq_b), Cv = pack2(sq_c, sq_c);
    int limcol = a.ncols - 1, lowcol = 0;   // columns kept for this row: lowcol <= col <= limcol
    if (a.mask) {
      if (rev) lowcol = row - a.off;
      else limcol = min(limcol, row + a.off);
    }
    const int wrow_lo = r0 + qd * 32, wrow_hi = wrow_lo + 31;
    float dl_row = 0.f;
    if (MODE == MODE_DQ && row_ok) dl_row = __ldg(a.dvec + (size_t)head * a.nrows + row);
    const uint64_t ndl_row = pack2(-dl_row, -dl_row);
    const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16);
    float* myvec = (float*)(smem + OFF_VEC) + warp * 64;
    const uint32_t myvec_s = sbase + OFF_VEC + warp * 256;
    // negated dvec of this lane's column in the warp's next tile, fetched one tile ahead
    auto fetch_vec = [&](int j, const ColPos& cp) -> float {
      const int col = tile_of(j, cp) * BN + cpart * 32 + lane;
      return (j < J && col < a.ncols) ? -__ldg(a.dvec + (size_t)head_of(cp) * a.ncols + col) : 0.f;
    };
    if (XT && J > 0) {
      // copy this warp's 32 rows x 16 bf16 pairs of x (warps 0-7) or u (warps 8-15) from the swizzled
      // row tile to TMEM: word c of a row is (element 2c, element 2c + 1), the A operand's layout
      if (!mbar_wait(BAR_X, 0)) report(11);
      const int cq = warp >> 2, r = qd * 32 + lane;
      const uint32_t src = sbase + (cq < 2 ? OFF_X : OFF_U) + r * 128;
      uint32_t xw[16];
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const ulonglong2 w2 = lds_v2(src + (((4 * (cq & 1) + v) ^ (r & 7)) << 4));
        xw[4 * v] = (uint32_t)w2.x; xw[4 * v + 1] = (uint32_t)(w2.x >> 32);
        xw[4 * v + 2] = (uint32_t)w2.y; xw[4 * v + 3] = (uint32_t)(w2.y >> 32);
      }
      tmem_st16(tl + T_X + cq * 16, xw);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR_XT);
    }
    ColPos pc = pos0;                     // position of this group's current tile
    advance(pc, gp);
    float nxt = rev ? fetch_vec(gp, pc) : 0.f;
    [[maybe_unused]] int hq_now = -1;
    uint64_t rs2[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};  // forward: row sum
    bool ok = true;
    for (int j = gp; j < J; j += 2, advance(pc, 2)) {
      const int i = j >> 1;
      const float cur = nxt;
      if (rev) {
        if constexpr (GQ) {
          ColPos pn = pc;                 // the group's next tile
          advance(pn, 2);
          nxt = fetch_vec(j + 2, pn);
        } else {
          nxt = fetch_vec(j + 2, pc);
        }
      }
      if constexpr (GQ) {
        if (rev && pc.h != hq_now) {   // the tile belongs to the next query head of the group
          hq_now = pc.h;
          const float cq = stat_scale(a.stat_q, pc.h, a.lim) * ck;
          const float B1 = a.a1 * cq, B2 = a.a2 * cq * cq;
          A1v = pack2(B1, B1);
          A2v = pack2(B2, B2);
          A2d = pack2(2.f * B2, 2.f * B2);
        }
      }
      // The group's previous products must have consumed E and P before they are overwritten.
      // grad_q waits for its S / W anyway (that path bounds its tile period), so the check goes
      // here, where it costs nothing on the way to the stores; the other two modes are bound by
      // their compute path and must not delay the S loads, so they check just before the stores.
      if (PV_EARLY && i > 0 && !mbar_wait(BAR_PV(gp), (uint32_t)((i - 1) & 1))) { report(9); ok = false; break; }
      const int set = j % kSets;                      // TRI: the tile's set
      const uint32_t tset = tl + set * SET_COLS;
      if (!mbar_wait(TRI ? BAR_TS(set) : BAR_S(gp), (uint32_t)((TRI ? j / kSets : i) & 1))) { report(7); ok = false; break; }
      tc_fence_after();
      const uint32_t vec_s = myvec_s + (i & 1) * 128;   // shared-window address of this tile's slot
      if (rev) {
        myvec[(i & 1) * 32 + lane] = cur;
        __syncwarp();
      }
      // the warp's HB columns in passes of 32
#pragma unroll
      for (int ps = 0; ps < HB / 32; ++ps) {
        uint32_t sv[32], wv[FWD ? 1 : 32];
        tmem_ld32(TRI ? tset + cpart * HB + ps * 32 : tl + T_S + gp * BN + cpart * HB + ps * 32, sv);
        if constexpr (!FWD) tmem_ld32(tl + T_W + gp * BN + cpart * HB + ps * 32, wv);
        tmem_wait_ld();
        if (!TRI && ps + 1 == HB / 32) {
          // S and W of this tile are in registers: the group's next tile may be issued
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_SFREE(gp));
        }
        const int c0 = tile_of(j, pc) * BN + cpart * HB + ps * 32;    // first of these 32 columns
        bool need_mask = (c0 + 32 > a.ncols);
        if (a.mask) need_mask = need_mask || (rev ? (c0 < wrow_hi - a.off) : (c0 + 31 > wrow_lo + a.off));
        // the mask test stays outside the element loops so that each loop is one basic block
        // whose sixteen independent pairs the compiler can interleave; E and P of a pair are
        // formed together so that S and W die pair by pair
        uint32_t pe[16], pp[FUSED ? 16 : 1];
        ulonglong2 nd2 = make_ulonglong2(0ull, 0ull);
        if constexpr (FWD) {
          if (!need_mask) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint64_t p2 = fma2(fma2(A2v, pack2u(sv[2 * e], sv[2 * e + 1]), A1v), pack2u(sv[2 * e], sv[2 * e + 1]), A0v);
              rs2[e & 3] = add2(rs2[e & 3], p2);
              pe[e] = pack_bf16_2(p2);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
              const int col = c0 + 2 * e;
              float v0, v1;
              unpack2(fma2(fma2(A2v, s2, A1v), s2, A0v), v0, v1);
              v0 = (col > limcol || col < lowcol) ? 0.f : v0;
              v1 = (col + 1 > limcol || col + 1 < lowcol) ? 0.f : v1;
              pe[e] = pack_bf16(v0, v1);
              // Tiles on the causal diagonal (and ragged last tiles) hold most of what an early row sees, so
              // their share of the row sum is taken from the ROUNDED values the product will use: numerator
              // and denominator then carry the same rounding, and a row with one key returns its value exactly.
              rs2[e & 3] = add2(rs2[e & 3], pack2(__uint_as_float(pe[e] << 16), __uint_as_float(pe[e] & 0xFFFF0000u)));
            }
          }
        } else if (!need_mask) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
            if (rev && (e & 1) == 0) nd2 = lds_v2(vec_s + (e >> 1) * 16);   // four column values per load
            const uint64_t ndl = rev ? ((e & 1) ? nd2.y : nd2.x) : ndl_row;
            if constexpr (SQ) {
              const uint64_t t2 = add2(s2, Bv);
              pe[e] = pack_bf16_2(mul2(t2, add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl)));
              pp[e] = pack_bf16_2(fma2(t2, t2, Cv));
            } else {
              pe[e] = pack_bf16_2(mul2(fma2(A2d, s2, A1v), add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl)));
              if (FUSED) pp[e] = pack_bf16_2(fma2(fma2(A2v, s2, A1v), s2, A0v));
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
            if (rev && (e & 1) == 0) nd2 = lds_v2(vec_s + (e >> 1) * 16);
            const uint64_t ndl = rev ? ((e & 1) ? nd2.y : nd2.x) : ndl_row;
            const int col = c0 + 2 * e;
            const bool z0 = col > limcol || col < lowcol, z1 = col + 1 > limcol || col + 1 < lowcol;
            float v0, v1;
            const uint64_t t2 = SQ ? add2(s2, Bv) : fma2(A2d, s2, A1v);
            unpack2(mul2(t2, add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl)), v0, v1);
            pe[e] = pack_bf16(z0 ? 0.f : v0, z1 ? 0.f : v1);
            if (FUSED) {
              unpack2(SQ ? fma2(t2, t2, Cv) : fma2(fma2(A2v, s2, A1v), s2, A0v), v0, v1);
              pp[e] = pack_bf16(z0 ? 0.f : v0, z1 ? 0.f : v1);
            }
          }
        }
        if (!TRI && !PV_EARLY && ps == 0 && i > 0) {
          if (!mbar_wait(BAR_PV(gp), (uint32_t)((i - 1) & 1))) { report(9); ok = false; break; }
          tc_fence_after();
        }
        // TRI: P over the first 16 of the 32 S columns this pass has just read
        tmem_st16(TRI ? tset + cpart * HB + ps * 32 : tl + T_E + gp * HB + cpart * (HB / 2) + ps * 16, pe);
        if constexpr (FUSED) tmem_st16(tl + T_P + gp * HB + cpart * (HB / 2) + ps * 16, pp);
      }
      if (!ok) break;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(TRI ? BAR_TP(set) : BAR_P(gp));
    }
    // ---- epilogue: 32 accumulator columns per warp ----
    if (ok && J > 0) {
      if (!mbar_wait(BAR_DONE, 0)) { report(10); ok = false; }
    }
    tc_fence_after();
    const int part4 = warp >> 2;
    float scale = 1.f, rowsum = 0.f;
    if (FWD && J > 0) {
      // a row's sum is spread over the four warps that share its TMEM lane quarter; every
      // compute warp reaches this barrier, whatever happened before
      float lo, hi;
      unpack2(add2(add2(rs2[0], rs2[1]), add2(rs2[2], rs2[3])), lo, hi);
      myvec[lane] = lo + hi;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      const float* parts = (const float*)(smem + OFF_VEC) + qd * 64 + lane;
      rowsum = (parts[0] + parts[4 * 64]) + (parts[8 * 64] + parts[12 * 64]);
      if (a.den_add && row_ok) rowsum += a.den_add[(size_t)head * a.nrows + row];
      scale = 1.0f / rowsum;
    }
    if (ok && J > 0 && (FUSED || part4 < 2)) {
      const size_t grow = (size_t)head * a.nrows + (row_ok ? row : 0);
      const bool second = FUSED && part4 >= 2;          // grad_v columns
      const int cc = (part4 & 1) * 32;
      const bool dots_here = !FWD && !second && a.dots != nullptr;
      const float* add = second ? a.o2_add : a.o_add;
      const float pre = SQ ? (second ? A2 : 2.f * A2) : 1.f;   // completed square: the factor left out of E' and P'
      const size_t orow = FWD ? out_row(head, row_ok ? row : 0, a.nrows, a.o_heads) : grow;
      const float part = store_row<32>(tl + (second ? T_O2 : T_O) + cc, row_ok,
                                       (__nv_bfloat16*)(second ? a.o2 : a.o) + orow * D + cc,
                                       add ? add + grow * D + cc : nullptr,
                                       dots_here ? (const __nv_bfloat16*)a.x + grow * D + cc : nullptr, scale, pre);
      if (FWD && part4 == 0 && row_ok) a.den_out[grow] = rowsum;
      if (dots_here) {
        float sum = part;
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        if (lane == 0) atomicAdd(a.dots + head, sum);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int MODE>
int launch_wide(const Ctx& c, const char* name, const void* x, const void* u, const void* y,
                const void* z, int nrows, int ncols, WArgs a) {
  // rows are key/value heads in MODE_DKDV and query heads otherwise; the columns are the other kind
  const int heads = (MODE == MODE_DKDV) ? c.p.bhkv : c.p.bh;
  const int col_heads = (MODE == MODE_DKDV) ? c.p.bh : c.p.bhkv;
  const int kv_ratio = c.p.bh / c.p.bhkv;
  if (heads == 0 || nrows == 0) return FASTMAX_OK;
  CUtensorMap tx, tu, ty, tz;
  int rc;
  if ((rc = tma_map_bf16(&tx, x, heads, nrows, D, BM))) return rc;
  if ((rc = tma_map_bf16(&tu, u ? u : x, heads, nrows, D, BM))) return rc;
  if ((rc = tma_map_bf16(&ty, y, col_heads, ncols, D, WCfg<MODE>::BN))) return rc;
  if ((rc = tma_map_bf16(&tz, z, col_heads, ncols, D, WCfg<MODE>::BN))) return rc;
  a.nrows = nrows;
  a.ncols = ncols;
  a.x = x;
  a.ntr = (nrows + BM - 1) / BM;
  dim3 grid((unsigned)((size_t)heads * a.ntr));
  if (MODE == MODE_DKDV && kv_ratio == 1 && a.a2 > 0.f) {
    FM_CUDA_TRY(cudaFuncSetAttribute(dense_tc_wide_kernel<MODE, false, MODE == MODE_DKDV>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, WCfg<MODE>::SMEM));
    FM_LAUNCH(name, c.stream,
              (dense_tc_wide_kernel<MODE, false, MODE == MODE_DKDV><<<grid, kThreads, WCfg<MODE>::SMEM, c.stream>>>(
                  tx, tu, ty, tz, a, kv_ratio)));
  } else if (kv_ratio > 1) {
    FM_CUDA_TRY(cudaFuncSetAttribute(dense_tc_wide_kernel<MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     WCfg<MODE>::SMEM));
    FM_LAUNCH(name, c.stream,
              (dense_tc_wide_kernel<MODE, true><<<grid, kThreads, WCfg<MODE>::SMEM, c.stream>>>(tx, tu, ty, tz, a, kv_ratio)));
  } else {
    FM_CUDA_TRY(cudaFuncSetAttribute(dense_tc_wide_kernel<MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     WCfg<MODE>::SMEM));
    FM_LAUNCH(name, c.stream,
              (dense_tc_wide_kernel<MODE, false><<<grid, kThreads, WCfg<MODE>::SMEM, c.stream>>>(tx, tu, ty, tz, a, kv_ratio)));
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace

// bf16, head dimension 64, bh a multiple of bhkv (grouped k/v heads are handled in the kernels);
// FASTMAX_B200_NO_WIDE=1 in the environment keeps the three-kernel backward.
bool dense_tc_wide_supports(const fastmax_problem& p) {
  static const bool off = [] {
    const char* e = getenv("FASTMAX_B200_NO_WIDE");
    return e && e[0] == '1';
  }();
  return !off && p.dtype == FASTMAX_BF16 && p.d == 64 && p.bhkv > 0 && p.bh % p.bhkv == 0;
}

int dense_tc_wide_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                           const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                           void* grad_k, void* grad_v, const ChunkAdd* ca) {
  const fastmax_problem& p = c.p;
  WArgs a = {};
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.off = p.nk - p.nq;
  a.mask = p.mask;
  a.a0 = p.a0;
  a.a1 = p.a1;
  a.a2 = (p.p == 2) ? p.a2 : 0.f;
  a.lim = p.lim;
  a.dvec = dvec;
  if (ca) a.chunk = ca->chunk;
  int rc;
  // grad_q: rows = queries, columns = keys
  a.o = grad_q;
  a.dots = p.normalize ? dots : nullptr;
  a.o_add = ca ? ca->gq_add : nullptr;
  if ((rc = launch_wide<MODE_DQ>(c, "fm_dense_tc_dq", q, gs, k, v, p.nq, p.nk, a))) return rc;
  // grad_k and grad_v: rows = keys, columns = queries
  a.o = grad_k;
  a.o2 = grad_v;
  a.dots = p.normalize ? dots + p.bh : nullptr;
  a.o_add = ca ? ca->gk_add : nullptr;
  a.o2_add = ca ? ca->gv_add : nullptr;
  return launch_wide<MODE_DKDV>(c, "fm_dense_tc_dkdv", k, v, q, gs, p.nk, p.nq, a);
}

int dense_tc_wide_forward(const Ctx& c, const void* q, const void* k, const void* v, const stat_t* stats,
                          void* out, float* den, const ChunkAdd* ca) {
  const fastmax_problem& p = c.p;
  WArgs a = {};
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.off = p.nk - p.nq;
  a.mask = p.mask;
  a.a0 = p.a0;
  a.a1 = p.a1;
  a.a2 = (p.p == 2) ? p.a2 : 0.f;
  a.lim = p.lim;
  a.o = out;
  a.den_out = den;
  a.o_heads = c.out_heads;
  if (ca) { a.chunk = ca->chunk; a.o_add = ca->out_add; a.den_add = ca->den_add; }
  return launch_wide<MODE_FWD>(c, "fm_dense_tc_fwd", q, nullptr, k, v, p.nq, p.nk, a);
}

int tc_wide_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_wtc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}
int tc_wide_status_reset(cudaStream_t stream) {
  const int zero = 0;
  FM_CUDA_TRY(cudaMemcpyToSymbolAsync(g_wtc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}


}  // namespace fm
