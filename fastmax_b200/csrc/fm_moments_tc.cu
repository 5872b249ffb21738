// Second-order part of the moment-state form on the tcgen05 tensor cores (bf16
// operands, fp32 accumulation), head dimension 64.  Two kernels:
//
// readout  -- for a tile of 128 tokens x and a prefix state S2[a][b][c] (symmetric in
//   a, b; c = 0..63 value columns, c = 64 the normaliser column):
//       T[i][c][b] = sum_a x_i[a] S2[a][b][c]                   tensor cores
//       type A:  r_i[c] = A2   sum_b x_i[b] T[i][c][b]          (numerator | denominator, grad_v)
//       type B:  r_i[b] = 2 A2 sum_c ut_i[c] T[i][c][b]         (grad_q, grad_k)
//   The state is read as bf16 rows (c*64 + b) of 64 a-values -- a K-major B operand
//   streamed by TMA -- and T never leaves the SM: each 128-column slice of it is
//   produced in tensor memory and contracted by the CUDA cores straight from there.
//   This replaces the d*d-wide feature contraction of the reference
//   (`old stuff/fastmax_cuda_forward_quad.cu`:111-135, 240-268 and the matching
//   backward loops) by a GEMM of the raw token tile against the state.
//
// state    -- T2[(a,b)][c] = sum_j y_j[a] y_j[b] z_j[c] over the tokens of a chunk: the
//   features y_a y_b (each unordered pair once) are formed on the CUDA cores and written
//   to tensor memory as the A operand, the value tile is the MN-major B operand delivered
//   by TMA, and the accumulators stay in tensor memory for the whole chunk.
//
// The normaliser column of the state build is a third, small tensor-core kernel here; the
// first-order and constant rows of the state stay on the kernels of fm_first_tc.cu and
// fm_moments_ffma.cu.
#include <cstdlib>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_mtc_status = 0;  // first protocol error seen by a kernel of this file

namespace {
using namespace sm100;

constexpr int D = 64;
constexpr int NROWS_T = 65 * 64;          // rows (c, b) of the transposed bf16 state
constexpr int NROWS_TP = 34 * 128;        // the first-order blocks (see first_rows_to_bf16t) and padding to whole 128-row tiles

__device__ __forceinline__ void report(int code) { atomicCAS(&g_mtc_status, 0, code); }
// 16 bytes from / 4 bytes to shared memory by shared-window address (keeps the access off the generic path)
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 r;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(saddr));
  return r;
}
__device__ __forceinline__ void sts32(uint32_t saddr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}

// =====================================================================================
// readout
// =====================================================================================
struct RtArgs {
  const void* x;       // (heads, n, 64) bf16 tokens
  const void* u;       // type B: (heads, n, 64) bf16 second operand (gs or v)
  const float* uvec;   // type B: (heads, n) dvec, whose negative is the 65th entry of ut; null = 1
  float* out_a;        // type A result (heads, n, 64) fp32
  float* den_a;        // type A normaliser column (heads, n), may be null
  float* out_b;        // type B result (heads, n, 64) fp32
  const stat_t* stat_q;
  const stat_t* stat_k;
  float a2, lim;
  int n, chunk, nchunk, state_per_chunk;
  int wide_io;         // out_a / out_b are 32-byte aligned
  int zero_chunk;      // tokens of this chunk read an empty state: zeros are written, nothing is multiplied (-1: none)
  // Type A also adds the first-order and constant terms when state_f32 is given: x . S1 comes out of the last
  // slice (the copy's rows 65*64..), the constant row and S1's normaliser column are read from the fp32 state.
  const float* state_f32;
  size_t per_state;
  int dvp;
  float a0, a1;
  // Type B does the same with one more slice: u . S1[a][0..63] from the tensor core (the copy's rows 66*64..,
  // the u tile as the A operand) plus e * S1[a][64] from the fp32 state.
  int first_b;
  int mode;            // 0: type A on two token tiles, 1: type B on two token tiles,
                       // 2: one token tile, group 0 type A and group 1 type B
};

constexpr int RT_THREADS = 352;   // warps 0-3 group 0, 4-7 group 1, 8 TMA producer, 9 and 10 MMA issuers
constexpr int RT_NS = 4;          // state-tile ring stages
constexpr int RT_TILE = 128 * D * 2;
constexpr int RT_OFF_X = 0;                         // two token tiles
constexpr int RT_OFF_ST = 2 * RT_TILE;              // ring
constexpr int RT_OFF_U = RT_OFF_ST + RT_NS * RT_TILE;    // two u tiles (type B with the first-order slice)
constexpr int RT_OFF_UT = RT_OFF_U + 2 * RT_TILE;        // [2][128][66] fp32 (type B operand rows)
constexpr int RT_UT_LD = 66;
constexpr int RT_OFF_BAR = RT_OFF_UT + 2 * 128 * RT_UT_LD * 4;
constexpr int RT_NBAR = 1 + 2 * RT_NS + 8;
constexpr int RT_OFF_TMEM = RT_OFF_BAR + RT_NBAR * 8;
constexpr int RT_OFF_VEC = RT_OFF_TMEM + 16;        // per type-A group: constant row [65] | S1 normaliser column [64]
constexpr int RT_VEC = 132;
constexpr int RT_SMEM = RT_OFF_VEC + 2 * RT_VEC * 4 + 1024;
constexpr int RT_NT = 33;                           // slices of 128 columns of T; slice 33 is type B's first-order one

__global__ void __launch_bounds__(RT_THREADS, 1)
readout_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmS,
                  const __grid_constant__ CUtensorMap tmU, const RtArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + RT_OFF_BAR;
  // barriers: x | st_full[NS] | st_empty[NS] | t_full[tile][buf] (4) | t_free[tile][buf] (4)
  auto BAR_X = [&]() { return bar0; };
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (1 + s); };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (1 + RT_NS + s); };
  auto BAR_TFULL = [&](int t, int b) { return bar0 + 8u * (1 + 2 * RT_NS + t * 2 + b); };
  auto BAR_TFREE = [&](int t, int b) { return bar0 + 8u * (5 + 2 * RT_NS + t * 2 + b); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + RT_OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_per_cta = (a.mode == 2) ? 1 : 2;
  const int ctas_per_head = (a.n + 128 * tiles_per_cta - 1) / (128 * tiles_per_cta);
  const int head = blockIdx.x / ctas_per_head;
  const int tok0 = (blockIdx.x % ctas_per_head) * 128 * tiles_per_cta;
  const int ntile = (tiles_per_cta == 2 && tok0 + 128 < a.n) ? 2 : 1;   // token tiles that have rows
  const int chunk = a.state_per_chunk ? tok0 / a.chunk : 0;
  const int srow = head * (a.state_per_chunk ? a.nchunk : 1) + chunk;   // index of the state matrix
  const int readers = (a.mode == 2) ? 8 : 4;                            // warps that read each T buffer
  const int nslice = RT_NT + (a.first_b ? 1 : 0);
  if (a.state_per_chunk && chunk == a.zero_chunk) {
    // the whole CTA lies in one chunk (chunks are multiples of 256 tokens): zero rows, no products
    const int rows = min(128 * tiles_per_cta, a.n - tok0);
    for (int i = tid; i < rows * (D / 4); i += RT_THREADS) {
      const size_t e = ((size_t)head * a.n + tok0) * D + (size_t)i * 4;
      if (a.mode != 1) *(float4*)(a.out_a + e) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a.mode != 0) *(float4*)(a.out_b + e) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.mode != 1 && a.den_a)
      for (int i = tid; i < rows; i += RT_THREADS) a.den_a[(size_t)head * a.n + tok0 + i] = 0.f;
    return;
  }

  if (tid == 0) {
    mbar_init(BAR_X(), 1);
    for (int s = 0; s < RT_NS; ++s) { mbar_init(BAR_FULL(s), 1); mbar_init(BAR_EMPTY(s), a.mode == 2 ? 1 : ntile); }
    for (int t = 0; t < 2; ++t)
      for (int b = 0; b < 2; ++b) { mbar_init(BAR_TFULL(t, b), 1); mbar_init(BAR_TFREE(t, b), readers); }
    mbar_fence_init();
  }
  if (warp == 9) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ---------------- TMA producer: token tiles once, then the 33 state tiles ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmS);
      mbar_expect_tx(BAR_X(), (a.first_b ? 2 : 1) * ntile * RT_TILE);
      for (int t = 0; t < ntile; ++t) tma_load_3d(sbase + RT_OFF_X + t * RT_TILE, &tmX, BAR_X(), 0, tok0 + t * 128, head);
      if (a.first_b) {
        tma_prefetch_desc(&tmU);
        for (int t = 0; t < ntile; ++t) tma_load_3d(sbase + RT_OFF_U + t * RT_TILE, &tmU, BAR_X(), 0, tok0 + t * 128, head);
      }
    }
    for (int n = 0; n < nslice; ++n) {
      const int s = n % RT_NS;
      if (!mbar_wait(BAR_EMPTY(s), (((n / RT_NS) & 1) ^ 1))) { report(21); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), RT_TILE);
        tma_load_3d(sbase + RT_OFF_ST + s * RT_TILE, &tmS, BAR_FULL(s), 0, n * 128, srow);
      }
    }
  } else if (warp >= 9) {
    // ---------------- MMA issuers: the whole warp runs the loop, one elected lane issues ----------------
    // Two warps, so that the barrier checks of one overlap the products of the other (the
    // tensor pipe's queue is short: a single issuer leaves it idle between slices).  With two
    // token tiles issuer w owns tile w; with one tile the issuers take alternate slices, so
    // each owns one T buffer and the ring stages of its parity.
    const int w = warp - 9;
    const bool one_tile = a.mode == 2;
    if (one_tile || w < ntile) {
      constexpr uint32_t idesc = idesc_bf16(128, 128, 0, 0);
      bool ok = mbar_wait_warp(BAR_X(), 0);
      if (!ok) report(22);
      tc_fence_after();
      const uint32_t st0 = desc_lo(sbase + RT_OFF_ST, 16);
      const int t = one_tile ? 0 : w;
      const uint32_t x_lo = desc_lo(sbase + RT_OFF_X + t * RT_TILE, 16);
      const uint32_t u_lo = desc_lo(sbase + RT_OFF_U + t * RT_TILE, 16);
      for (int n = one_tile ? w : 0; ok && n < nslice; n += one_tile ? 2 : 1) {
        const int s = n % RT_NS, buf = n & 1;
        if (!mbar_wait_warp(BAR_FULL(s), (uint32_t)((n / RT_NS) & 1))) { report(23); break; }
        // the buffer was last used by slice n-2
        if (n >= 2 && !mbar_wait_warp(BAR_TFREE(t, buf), (uint32_t)(((n >> 1) - 1) & 1))) { report(24); break; }
        tc_fence_after();
        if (elect_one()) {
          umma_ss_k64(tmem + t * 256 + buf * 128, n < RT_NT ? x_lo : u_lo, st0 + (uint32_t)s * (RT_TILE >> 4), idesc);
          umma_commit(BAR_TFULL(t, buf));
          umma_commit(BAR_EMPTY(s));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ---------------- contraction groups ----------------
    const int g = warp >> 2, qd = warp & 3;
    const int t = (a.mode == 2) ? 0 : g;                 // token tile this group reads
    const bool type_b = (a.mode == 1) || (a.mode == 2 && g == 1);
    if (t < ntile) {
      const int tok = tok0 + t * 128 + qd * 32 + lane;
      const bool tok_ok = tok < a.n;
      const size_t grow = (size_t)head * a.n + (tok_ok ? tok : 0);
      const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head, a.lim);
      const float A2 = a.a2 * c * c;
      const uint32_t tbase = tmem + t * 256 + ((uint32_t)(qd * 32) << 16);
      // 32 packed fp32 pairs per thread: type A keeps its token row here, type B its 64 running sums
      // (one array for both, so that neither kind carries the other's registers through the loop)
      uint64_t xa[32];
      if (!type_b) {
        const uint4* xr = (const uint4*)((const __nv_bfloat16*)a.x + grow * D);
#pragma unroll
        for (int v8 = 0; v8 < 8; ++v8) {
          uint4 w = tok_ok ? __ldg(xr + v8) : make_uint4(0, 0, 0, 0);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            xa[v8 * 4 + e] = pack2(__uint_as_float(ww[e] << 16), __uint_as_float(ww[e] & 0xFFFF0000u));
        }
      }
      float* ut = (float*)(smem + RT_OFF_UT) + ((size_t)g * 128 + qd * 32 + lane) * RT_UT_LD;
      if (type_b) {
        // ut row = [u_0 .. u_63 | e]; only this thread reads it back
        const uint4* ur = (const uint4*)((const __nv_bfloat16*)a.u + grow * D);
#pragma unroll
        for (int v8 = 0; v8 < 8; ++v8) {
          uint4 w = tok_ok ? __ldg(ur + v8) : make_uint4(0, 0, 0, 0);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            ut[v8 * 8 + 2 * e] = __uint_as_float(ww[e] << 16);
            ut[v8 * 8 + 2 * e + 1] = __uint_as_float(ww[e] & 0xFFFF0000u);
          }
        }
        ut[64] = tok_ok ? (a.uvec ? -a.uvec[grow] : 1.0f) : 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) xa[e] = pack2(0.f, 0.f);
      }
      const bool first_too = !type_b && a.state_f32 != nullptr;
      const bool first_b = type_b && a.first_b != 0;
      const float A1f = a.a1 * c;
      float k_out = 2.f * A2;                                  // type B: factor of the running sums at the end
      float* vec = (float*)(smem + RT_OFF_VEC) + g * RT_VEC;   // crow[0..64] | ncol[0..63]
      if (first_too || first_b) {
        // the group's 128 threads stage the two vectors of this CTA's state (all of them reach the barrier:
        // a group is of one kind)
        const float* fs = a.state_f32 + (size_t)srow * a.per_state + (size_t)(64 * 64) * a.dvp;   // first-order rows
        const int i = qd * 32 + lane;
        if (i < 65) vec[i] = __ldg(fs + (size_t)64 * a.dvp + i);               // constant row
        if (i < 64) vec[65 + i] = __ldg(fs + (size_t)i * a.dvp + 64);           // S1[a][64]
        if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      bool ok = true;
      for (int n = 0; n < nslice; ++n) {
        const int buf = n & 1;
        if (n == RT_NT && !type_b) break;     // the last slice is type B's alone (nothing waits for its release)
        if (!mbar_wait(BAR_TFULL(t, buf), (uint32_t)((n >> 1) & 1))) { report(25); ok = false; break; }
        tc_fence_after();
        if (n == RT_NT) {
          // first-order slice: T1[a] = u . S1[a][0..63] in the first 64 columns; the running sums take their
          // final factor here and the first-order term joins them
          uint32_t tv[64];
          tmem_ld64(tbase + buf * 128, tv);
          tmem_wait_ld();
          const float ue = ut[64];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float f0, f1;
            unpack2(xa[e], f0, f1);
            f0 = fmaf(k_out, f0, A1f * fmaf(ue, vec[65 + 2 * e], __uint_as_float(tv[2 * e])));
            f1 = fmaf(k_out, f1, A1f * fmaf(ue, vec[66 + 2 * e], __uint_as_float(tv[2 * e + 1])));
            xa[e] = pack2(f0, f1);
          }
          k_out = 1.f;
          break;
        }
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int cidx = 2 * n + hf;       // column c of the state this half belongs to
          uint32_t tv[64];
          tmem_ld64(tbase + buf * 128 + hf * 64, tv);
          tmem_wait_ld();
          if (hf == 1) {                      // both halves are in registers or consumed: release
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_TFREE(t, buf));
          }
          if (cidx > 64) {                    // the last 64 rows of the copy: the first-order block
            if (first_too) {
              // T1[c] = x . S1[:, c] in this half; the normaliser column's first-order part is a dot on the CUDA cores
#pragma unroll
              for (int cc = 0; cc < 64; ++cc) ut[cc] += fmaf(A1f, __uint_as_float(tv[cc]), a.a0 * vec[cc]);
              uint64_t s4[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
              for (int e = 0; e < 32; ++e) s4[e & 3] = fma2(xa[e], pack2(vec[65 + 2 * e], vec[66 + 2 * e]), s4[e & 3]);
              float lo, hi;
              unpack2(add2(add2(s4[0], s4[1]), add2(s4[2], s4[3])), lo, hi);
              ut[64] += fmaf(A1f, lo + hi, a.a0 * vec[64]);
            }
            continue;
          }
          if (!type_b) {
            uint64_t s4[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
            for (int e = 0; e < 32; ++e) s4[e & 3] = fma2(xa[e], pack2u(tv[2 * e], tv[2 * e + 1]), s4[e & 3]);
            float lo, hi;
            unpack2(add2(add2(s4[0], s4[1]), add2(s4[2], s4[3])), lo, hi);
            ut[cidx] = A2 * (lo + hi);      // staged in this thread's row, written out at the end
          } else {
            const float uc = ut[cidx];
            const uint64_t u2 = pack2(uc, uc);
#pragma unroll
            for (int e = 0; e < 32; ++e) xa[e] = fma2(u2, pack2u(tv[2 * e], tv[2 * e + 1]), xa[e]);
          }
        }
      }
      if (ok && !type_b && tok_ok) {
        // a thread owns its 256-byte row: 32-byte stores write whole sectors
        float* dst = a.out_a + grow * D;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          uint32_t w[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) w[q] = __float_as_uint(ut[8 * e + q]);
          stg32(dst + 8 * e, w, a.wide_io != 0);
        }
        if (a.den_a) a.den_a[grow] = ut[64];
      }
      if (ok && type_b && tok_ok) {
        const float k2 = k_out;
        float* dst = a.out_b + grow * D;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          uint32_t w[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float f0, f1;
            unpack2(xa[4 * e + q], f0, f1);
            w[2 * q] = __float_as_uint(k2 * f0);
            w[2 * q + 1] = __float_as_uint(k2 * f1);
          }
          stg32(dst + 8 * e, w, a.wide_io != 0);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =====================================================================================
// bf16 transposed copy of the second-order block of fp32 prefix states:
//   out[m][c*64 + b][a] = state[m][(b*64 + a)][c]      (S2 is symmetric in a, b)
// one CTA per (state matrix m, b).  The 64 rows past 65*64 hold the first-order block the same way,
//   out[m][65*64 + c][a] = state[m][64*64 + a][c],  c < 64
// so that the read-out's last slice yields x . S1 beside the normaliser column's second-order part, and the
// 64 rows after those hold it untransposed,
//   out[m][66*64 + a][c] = state[m][64*64 + a][c],  c < 64
// the B operand of type B's first-order slice (u . S1[a][:]).  The remaining 64 rows of the last tile are
// never written; the columns of T they produce are never read.
// =====================================================================================
// rows 65*64 .. 65*64 + 63 of one copy from the (summed) first-order rows of its fp32 state
__device__ __forceinline__ void first_rows_to_bf16t(const float* __restrict__ st, __nv_bfloat16* __restrict__ o,
                                                    int dvp, float (*blk)[69], int t) {
  const float* src = st + (size_t)64 * 64 * dvp;     // rows 4096 + a, a = 0..63
  for (int i = t; i < 64 * dvp; i += 256) blk[i / dvp][i % dvp] = src[i];
  __syncthreads();
  uint32_t* ow = (uint32_t*)(o + (size_t)NROWS_T * 64);
  for (int w = t; w < 64 * 32; w += 256) {
    const int cc = w >> 5, ap = (w & 31) * 2;
    ow[64 * 32 + w] = pack_bf16(blk[cc][ap], blk[cc][ap + 1]);     // rows 66*64 + a: S1[a][c], c contiguous (type B)
    ow[cc * 32 + (w & 31)] = pack_bf16(blk[ap][cc], blk[ap + 1][cc]);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256) state_to_bf16t_kernel(const float* __restrict__ state,
                                                             __nv_bfloat16* __restrict__ out, int dvp,
                                                             size_t per_state) {
  __shared__ float blk[64][69];
  const int m = blockIdx.y, b = blockIdx.x;
  if (b == 64) {  // the first-order rows (the fp32 state holds running sums already)
    first_rows_to_bf16t(state + (size_t)m * per_state, out + (size_t)m * NROWS_TP * 64, dvp, blk, threadIdx.x);
    return;
  }
  const float* src = state + (size_t)m * per_state + (size_t)b * 64 * dvp;   // rows (b, a = 0..63)
  for (int i = threadIdx.x; i < 64 * dvp; i += 256) blk[i / dvp][i % dvp] = src[i];
  __syncthreads();
  __nv_bfloat16* o = out + (size_t)m * NROWS_TP * 64;
  for (int i = threadIdx.x; i < 65 * 64; i += 256) {
    const int c = i / 64, aa = i % 64;
    o[((size_t)c * 64 + b) * 64 + aa] = __float2bfloat16_rn(blk[aa][c]);
  }
}

// =====================================================================================
// Running sum over the chunks of a head and the bf16 transposed copy in one pass, second-order
// rows only:  out[m][c*64 + b][a] = bf16( base[(b*64 + a)][c] + sum of state[m'][(b*64 + a)][c] over
// the chunks m' before m (after m when reverse) ).  One CTA per (head, b) keeps its 64 x 68 block of
// the running sum in registers, in fp32, walks the chunks in order and reads every raw chunk state
// once; the fp32 states are left as they are.  The block with b == 64 copies the first-order rows
// (already summed in place) into the last 64 rows of every copy.
// =====================================================================================
__global__ void __launch_bounds__(256) prefix_bf16t_kernel(const float* __restrict__ state,
                                                           const float* __restrict__ base,
                                                           __nv_bfloat16* __restrict__ out, int nchunk, int dvp,
                                                           size_t per_state, int reverse) {
  __shared__ float blk[64][69];
  const int head = blockIdx.y, b = blockIdx.x, t = threadIdx.x;
  if (b == 64) {
    // the first-order rows: their running sums were formed in place in the fp32 states before this launch
    for (int i = 0; i < nchunk; ++i)
      first_rows_to_bf16t(state + (size_t)(head * nchunk + i) * per_state,
                          out + (size_t)(head * nchunk + i) * NROWS_TP * 64, dvp, blk, t);
    return;
  }
  constexpr int NV = 64 * 68 / 4;                    // float4 pieces of the block (dvp == 68)
  const size_t blk_off = (size_t)b * 64 * dvp;       // rows (b, a = 0..63) are contiguous
  float4 run[5], nxt[5];
#pragma unroll
  for (int u = 0; u < 5; ++u) {
    const int v = t + u * 256;
    run[u] = (base && v < NV) ? *(const float4*)(base + (size_t)head * per_state + blk_off + 4 * v)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  auto load = [&](int i, float4 (&r)[5]) {
    const int c = reverse ? nchunk - 1 - i : i;
    const float* src = state + (size_t)(head * nchunk + c) * per_state + blk_off;
#pragma unroll
    for (int u = 0; u < 5; ++u) {
      const int v = t + u * 256;
      // the last chunk in scan order is never added to anything that is written (and may not have been built)
      r[u] = (i + 1 < nchunk && v < NV) ? __ldcs((const float4*)(src + 4 * v)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  load(0, nxt);
  for (int i = 0; i < nchunk; ++i) {
    const int c = reverse ? nchunk - 1 - i : i;
    // the exclusive running sum of this chunk, transposed through shared memory
#pragma unroll
    for (int u = 0; u < 5; ++u) {
      const int v = t + u * 256;
      if (v < NV) {
        const int e = 4 * v, aa = e / 68, cc = e % 68;   // 68 is a multiple of 4: a piece never straddles rows
        blk[aa][cc] = run[u].x; blk[aa][cc + 1] = run[u].y; blk[aa][cc + 2] = run[u].z; blk[aa][cc + 3] = run[u].w;
      }
    }
    float4 cur[5];
#pragma unroll
    for (int u = 0; u < 5; ++u) cur[u] = nxt[u];
    load(i + 1, nxt);                                  // in flight during the transposed write
    __syncthreads();
    uint32_t* o = (uint32_t*)(out + (size_t)(head * nchunk + c) * NROWS_TP * 64);
    for (int w = t; w < 65 * 32; w += 256) {
      const int cc = w >> 5, ap = (w & 31) * 2;
      o[((size_t)cc * 64 + b) * 32 + (w & 31)] = pack_bf16(blk[ap][cc], blk[ap + 1][cc]);
    }
#pragma unroll
    for (int u = 0; u < 5; ++u) {
      run[u].x += cur[u].x; run[u].y += cur[u].y; run[u].z += cur[u].z; run[u].w += cur[u].w;
    }
    __syncthreads();
  }
}

// =====================================================================================
// state build: T2[(a,b)][c] = sum_j y_j[a] y_j[b] z_j[c],  c < 64
// T2 is symmetric in (a, b), so each of the 2080 unordered pairs is formed once and its row is
// written to both of its places: 17 tiles of 128 pairs instead of 32 tiles of ordered ones.
// Five CTAs share one chunk of one head; four own four accumulator tiles of 128 pairs by 64
// columns (TMEM columns 0..255), the fifth one tile (see the pair table in the kernel), and each
// walks the chunk in blocks of 128 tokens.  The feature tiles are the A operand and live in
// tensor memory, never in shared memory: a TMEM lane of tile m holds its pair's product
// y[b] y[other] for the block's 128 tokens as 64 packed bf16 pairs (columns 256 + 64 m ..),
// written by the threads that own the lane, and the value tile that TMA delivered is the
// MN-major B operand of eight K=16 products per tile.
//   The sixteen generator warps form two independent halves, one per 64 tokens of the block
// (warps 0-7 and 8-15), each with its own named barrier, feature-buffer columns, mbarriers
// and MMA issuer warp, so that the latency chain of one half (transpose, barrier, row reads,
// TMEM stores, hand-off) overlaps that of the other.  A half first transposes its y rows
// into shared memory (yT[feature][token]), so that a thread reads its own row b once, as
// 16-byte vectors, and the tile's other row per tile (one row for the whole warp where the pair
// is feature x fixed feature, the warp's 32 rows rotated where it is a distance around the
// ring); warp w covers the TMEM lane quarter w % 4 and 32 tokens.  Shared-memory traffic per
// block is the transposition, the row reads and the tensor core's reads of the value tile, a
// fraction of what feature tiles staged in shared memory cost.  The y rows come straight from global memory into
// registers two blocks ahead; the producer warp asks for them in L2 earlier still.
// =====================================================================================
struct StArgs {
  const void* y;     // (heads, n, 64) bf16 feature source
  float* state;      // (heads, nchunk, F, DVP) fp32; rows a*64+b and b*64+a of each pair, columns 0..64 and padding
  int n, chunk, nchunk, dvp;
  size_t per_state;
  int skip_chunk;    // this chunk's state is not wanted (-1: none)
};

constexpr int ST_GEN_WARPS = 16;
constexpr int ST_THREADS = (ST_GEN_WARPS + 3) * 32;   // warps 0-15: generators; 16: TMA; 17, 18: MMA issuers
constexpr int ST_TILES = 4;           // accumulator tiles (and feature buffers) per CTA
constexpr int ST_SPLIT = 5;            // CTAs per (head, chunk): four of four tiles and one of one tile
constexpr int ST_NZ = 3;              // value-tile ring
constexpr int ST_ZTILE = 128 * 128;
constexpr int ST_YT_LD = 272;         // bytes per yT row: 128 tokens + 16 (conflict-free 16-byte reads down a column)
constexpr int ST_YT = 64 * ST_YT_LD;
constexpr int ST_OFF_Z = 0;
constexpr int ST_OFF_YT = ST_NZ * ST_ZTILE;          // two transposed blocks
constexpr int ST_OFF_BAR = ST_OFF_YT + 2 * ST_YT;
constexpr int ST_NBAR = 5 * ST_TILES + 2 * ST_NZ + 1;
constexpr int ST_OFF_TMEM = ST_OFF_BAR + ST_NBAR * 8;
constexpr int ST_SMEM = ST_OFF_TMEM + 16 + 1024;
constexpr int ST_TM_A = 64 * ST_TILES;               // first TMEM column of the feature buffers
constexpr int ST_L2_AHEAD = 5;                       // blocks between the L2 request and the use of y rows
static_assert(ST_TILES == 4 && ST_GEN_WARPS == 16, "the epilogue gives one tile to each group of four warps");

__global__ void __launch_bounds__(ST_THREADS, 1)
state_tc_kernel(const __grid_constant__ CUtensorMap tmZ, const StArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + ST_OFF_BAR;
  // barriers: a_full[tile][half] | a_empty[tile][half] | z_full[NZ] | z_empty[NZ] | done
  auto BAR_AFULL = [&](int m, int h) { return bar0 + 8u * (2 * m + h); };
  auto BAR_AEMPTY = [&](int m, int h) { return bar0 + 8u * (2 * ST_TILES + 2 * m + h); };
  auto BAR_ZFULL = [&](int s) { return bar0 + 8u * (4 * ST_TILES + s); };
  auto BAR_ZEMPTY = [&](int s) { return bar0 + 8u * (4 * ST_TILES + ST_NZ + s); };
  auto BAR_DONE = [&]() { return bar0 + 8u * (4 * ST_TILES + 2 * ST_NZ); };
  // completes once, when half 0's first product of tile m is done (a_empty[m][0] completes every block, and a
  // late waiter on one parity of it could see two completions as none)
  auto BAR_START = [&](int m) { return bar0 + 8u * (4 * ST_TILES + 2 * ST_NZ + 1 + m); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + ST_OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = blockIdx.x % ST_SPLIT;
  const int hc = blockIdx.x / ST_SPLIT;           // head * nchunk + chunk
  const int head = hc / a.nchunk, chunk = hc % a.nchunk;
  if (chunk == a.skip_chunk) return;
  const int t_begin = chunk * a.chunk, t_end = min(a.n, t_begin + a.chunk);
  const int nblk = (t_end - t_begin + 127) / 128;
  const int ntile = part == 4 ? 1 : ST_TILES;
  const __nv_bfloat16* ybase = (const __nv_bfloat16*)a.y + (size_t)head * a.n * D;

  if (tid == 0) {
    for (int m = 0; m < ST_TILES; ++m)
      for (int h = 0; h < 2; ++h) { mbar_init(BAR_AFULL(m, h), ST_GEN_WARPS / 2); mbar_init(BAR_AEMPTY(m, h), 1); }
    for (int m = 0; m < ST_TILES; ++m) mbar_init(BAR_START(m), 1);
    for (int s = 0; s < ST_NZ; ++s) { mbar_init(BAR_ZFULL(s), 1); mbar_init(BAR_ZEMPTY(s), 2); }
    mbar_init(BAR_DONE(), 2);
    mbar_fence_init();
  }
  if (warp == ST_GEN_WARPS + 1) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == ST_GEN_WARPS) {
    // ---- producer: value tiles by TMA, and L2 requests for the y rows of later blocks ----
    if (lane == 0) tma_prefetch_desc(&tmZ);
    auto ask_l2 = [&](int k) {
      if (k >= nblk) return;
      for (int i = lane; i < 128; i += 32) {
        const int tok = t_begin + k * 128 + i;
        if (tok < t_end) asm volatile("prefetch.global.L2 [%0];" ::"l"(ybase + (size_t)tok * D));
      }
    };
    for (int k = 2; k < ST_L2_AHEAD; ++k) ask_l2(k);
    for (int k = 0; k < nblk; ++k) {
      const int s = k % ST_NZ;
      ask_l2(k + ST_L2_AHEAD);
      if (!mbar_wait(BAR_ZEMPTY(s), (((k / ST_NZ) & 1) ^ 1))) { report(31); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_ZFULL(s), ST_ZTILE);
        // rows past the end of the sequence are zero-filled by TMA; rows past the end of the
        // chunk but inside the sequence are cancelled by zero features
        tma_load_3d(sbase + ST_OFF_Z + s * ST_ZTILE, &tmZ, BAR_ZFULL(s), 0, t_begin + k * 128, head);
      }
    }
  } else if (warp > ST_GEN_WARPS) {
    // Issuer warp w serves token half w of every block: the whole warp runs the loop, one elected
    // lane issues four K=16 products per tile.  Both halves add into the same accumulators; in the
    // first block half 1 lets half 0's product of a tile complete first, because that one starts
    // the accumulator.
    const int w = warp - ST_GEN_WARPS - 1;
    constexpr uint32_t idesc = idesc_bf16(128, 64, 0, 1);
    bool ok = true;
    for (int k = 0; ok && k < nblk; ++k) {
      const int s = k % ST_NZ;
      if (!mbar_wait_warp(BAR_ZFULL(s), (uint32_t)((k / ST_NZ) & 1))) { report(32); ok = false; break; }
      const uint32_t z_lo = desc_lo(sbase + ST_OFF_Z + s * ST_ZTILE, ST_ZTILE) + (uint32_t)w * (4 * 128);
      if (ntile == 1) {
        // one tile: its four feature buffers are a ring over blocks, so that the threads that form the
        // features run ahead of the products instead of waiting for each one
        const int fb = k & 3;
        if (!mbar_wait_warp(BAR_AFULL(fb, w), (uint32_t)((k >> 2) & 1))) { report(33); ok = false; break; }
        if (k == 0 && w == 1 && !mbar_wait_warp(BAR_START(0), 0)) { report(36); ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          umma_ts_steps<4>(tmem, tmem + ST_TM_A + fb * 64 + w * 32, z_lo, idesc, (k > 0 || w == 1) ? 1u : 0u);
          umma_commit(BAR_AEMPTY(fb, w));
          if (k == 0 && w == 0) umma_commit(BAR_START(0));
        }
        __syncwarp();
      } else
      for (int m = 0; m < ntile; ++m) {
        if (!mbar_wait_warp(BAR_AFULL(m, w), (uint32_t)(k & 1))) { report(33); ok = false; break; }
        if (k == 0 && w == 1 && !mbar_wait_warp(BAR_START(m), 0)) { report(36); ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          umma_ts_steps<4>(tmem + m * 64, tmem + ST_TM_A + m * 64 + w * 32, z_lo, idesc, (k > 0 || w == 1) ? 1u : 0u);
          umma_commit(BAR_AEMPTY(m, w));
          if (k == 0 && w == 0) umma_commit(BAR_START(m));
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(BAR_ZEMPTY(s));
      __syncwarp();
    }
    if (ok && elect_one()) umma_commit(BAR_DONE());
    __syncwarp();
  } else {
    const int h = warp >> 3, tq = (warp >> 2) & 1, qd = warp & 3;   // token half, 32-token quarter in it, TMEM lane quarter
    // This thread's lane of tile m holds the unordered pair {b, other(m)}: b is the thread's own feature
    // (the same in every tile, so its row is read once per block), other(m) the tile's.
    //   part 0: b = lane,      other = (lane + s) % 32,      s = 4 m + quarter = 0..15   (pairs inside features 0..31)
    //   part 1: b = 32 + lane, other = 4 m + quarter                                     (features 32..63 x 0..15)
    //   part 2: b = 32 + lane, other = 16 + 4 m + quarter                                (features 32..63 x 16..31)
    //   part 3: b = 32 + lane, other = 32 + (lane + s) % 32                              (pairs inside 32..63)
    //   part 4: one tile; quarter 0: b = lane, quarter 1: b = 32 + lane, other = b's partner at distance 16, of
    //           which lanes 0..15 are new pairs; quarters 2 and 3 repeat them and are not stored.
    // Distances 0..15 around the ring of 32 give every pair inside a group of 32 once, distance 16 gives the
    // remaining sixteen; 2080 pairs in 17 tiles of 128 lanes instead of 4096 ordered ones in 32.
    const int grp = part == 0 ? 0 : (part < 4 ? 1 : (qd & 1));
    const int b = grp * 32 + lane;
    const int o_off = (part == 3 || part == 4) ? grp * 32 : 0;
    const int o_sum = ((part == 1 || part == 2) ? 0 : lane) + (part == 4 ? 16 : (part == 2 ? 16 + qd : qd));
    auto other = [&](int m) { return o_off + ((o_sum + 4 * m) & 31); };
    const int tok_off = h * 64 + tq * 32;           // first of this warp's 32 tokens in the block
    // transposition duty inside the half: token pair jp (of 32) and 8 features from fg * 8
    const int jp = tid & 31, fg = (tid >> 5) & 7;
    auto load_rows = [&](int k, uint4 (&r)[2]) {
      const int tok = t_begin + k * 128 + h * 64 + 2 * jp;
#pragma unroll
      for (int t = 0; t < 2; ++t)
        r[t] = (k < nblk && tok + t < t_end) ? __ldg((const uint4*)(ybase + (size_t)(tok + t) * D + fg * 8))
                                             : make_uint4(0, 0, 0, 0);
    };
    uint4 rows[2], rows_next[2];
    load_rows(0, rows);
    load_rows(1, rows_next);
    const uint32_t ta = tmem + ST_TM_A + h * 32 + tq * 16 + ((uint32_t)(qd * 32) << 16);   // this warp's part of feature buffer 0
    bool ok = true;
    for (int k = 0; k < nblk; ++k) {   // every generator thread takes part in every block's barrier
      const uint32_t yt = sbase + ST_OFF_YT + (k & 1) * ST_YT;
      {
        // word (feature f, token pair) = two consecutive tokens of feature f
        const uint32_t t0[4] = {rows[0].x, rows[0].y, rows[0].z, rows[0].w};
        const uint32_t t1[4] = {rows[1].x, rows[1].y, rows[1].z, rows[1].w};
        const uint32_t col = yt + (fg * 8) * ST_YT_LD + (h * 32 + jp) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sts32(col + (2 * e) * ST_YT_LD, __byte_perm(t0[e], t1[e], 0x5410));
          sts32(col + (2 * e + 1) * ST_YT_LD, __byte_perm(t0[e], t1[e], 0x7632));
        }
      }
      rows[0] = rows_next[0];
      rows[1] = rows_next[1];
      load_rows(k + 2, rows_next);                  // two blocks ahead
      if (h == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
      // Reuse of a yT buffer two blocks later needs no second barrier: a thread that writes block
      // k + 2 has passed the barrier of block k + 1, which every thread of its half reaches only
      // after its reads of block k (a half reads only the token columns it wrote).
      if (!ok) continue;
      uint32_t yb[16];
      {
        const uint32_t rb = yt + b * ST_YT_LD + tok_off * 2;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 w4 = lds128(rb + v * 16);
          yb[4 * v] = w4.x; yb[4 * v + 1] = w4.y; yb[4 * v + 2] = w4.z; yb[4 * v + 3] = w4.w;
        }
      }
      // products of one tile: row a of the tile (a broadcast read) times this thread's row b
      auto products = [&](int m, uint32_t (&pr)[16]) {
        const uint32_t ra = yt + other(m) * ST_YT_LD + tok_off * 2;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 w4 = lds128(ra + v * 16);
          const uint32_t ya[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 pv = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&yb[4 * v + e]),
                                              *reinterpret_cast<const __nv_bfloat162*>(&ya[e]));
            pr[4 * v + e] = *reinterpret_cast<const uint32_t*>(&pv);
          }
        }
      };
      // Tiles go two at a time, and the stores of one pair complete while the products of the next
      // are formed.  A feature buffer is free once the product that read it one block ago is done;
      // products complete in order, so the later tile's barrier covers the earlier one's too.
      uint32_t p0[16], p1[16], p2[16], p3[16];
      products(0, p0);
      if (ntile == 1) {
        const int fb = k & 3;                       // feature buffer of this block (a ring over blocks)
        if (!mbar_wait(BAR_AEMPTY(fb, h), (uint32_t)(((k >> 2) & 1) ^ 1))) { report(34); ok = false; continue; }
        tc_fence_after();
        tmem_st16(ta + 64 * fb, p0);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_AFULL(fb, h));
        continue;
      }
      products(1, p1);
      if (!mbar_wait(BAR_AEMPTY(1, h), (uint32_t)((k & 1) ^ 1))) { report(34); ok = false; continue; }
      tc_fence_after();
      tmem_st16(ta, p0);
      tmem_st16(ta + 64, p1);
      products(2, p2);
      products(3, p3);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(BAR_AFULL(0, h)); mbar_arrive(BAR_AFULL(1, h)); }
      if (!mbar_wait(BAR_AEMPTY(3, h), (uint32_t)((k & 1) ^ 1))) { report(34); ok = false; continue; }
      tc_fence_after();
      tmem_st16(ta + 128, p2);
      tmem_st16(ta + 192, p3);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(BAR_AFULL(2, h)); mbar_arrive(BAR_AFULL(3, h)); }
    }
    // ---- epilogue: accumulator rows -> fp32 state (columns 0..63), the normaliser column from the
    // block state_ecol_tc_kernel left in the first-order rows, zero padding ----
    float* st = a.state + (size_t)hc * a.per_state;
    const int m = warp >> 2;                       // one tile per group of four warps
    const int o = other(m);
    const bool warp_mine = m < ntile && (part < 4 || qd < 2);   // the TMEM read is a whole-warp instruction
    const bool mine = warp_mine && (part < 4 || lane < 16);
    // column 64 of the pair's two rows (65..67 are padding, dvp == 68), asked for before the wait for the products
    uint32_t ecols[2] = {0u, 0u};
    if (ok && mine) {
      ecols[0] = __float_as_uint(st[(size_t)4096 * a.dvp + b * 64 + o]);
      ecols[1] = __float_as_uint(st[(size_t)4096 * a.dvp + o * 64 + b]);
    }
    if (ok && !mbar_wait(BAR_DONE(), 0)) { report(35); ok = false; }
    tc_fence_after();
    if (ok) {
      uint32_t tv[64];
      if (warp_mine) {
        tmem_ld64(tmem + m * 64 + ((uint32_t)(qd * 32) << 16), tv);
        tmem_wait_ld();
      }
      // the pair's row goes to both of its places in the state, (b, other) and (other, b)
      for (int side = 0; mine && side < (o == b ? 1 : 2); ++side) {
      const int f = side == 0 ? b * 64 + o : o * 64 + b;
      float* dst = st + (size_t)f * a.dvp;
      const uint32_t ecol = ecols[side];
      // A thread owns its 272-byte row, so its stores share no sector with its neighbours': 32-byte stores
      // (whole sectors) wherever the row allows.  A row that starts on a 32-byte boundary is 8 x 32 + 16
      // bytes, one that starts 16 bytes past a boundary is 16 + 8 x 32 (rows and matrices are 16-byte multiples).
      if (((uintptr_t)dst & 16) != 0) {
        *(float4*)dst = make_float4(__uint_as_float(tv[0]), __uint_as_float(tv[1]), __uint_as_float(tv[2]),
                                    __uint_as_float(tv[3]));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          uint32_t w[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int col = 4 + 8 * e + q;
            w[q] = col < 64 ? tv[col < 64 ? col : 0] : (col == 64 ? ecol : 0u);
          }
          stg32(dst + 4 + 8 * e, w, true);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          uint32_t w[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) w[q] = tv[8 * e + q];
          stg32(dst + 8 * e, w, true);
        }
        *(float4*)(dst + 64) = make_float4(__uint_as_float(ecol), 0.f, 0.f, 0.f);
      }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ST_GEN_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Normaliser column of the second-order rows on the tensor cores:
//   state[(a,b)][64] = E[a][b] = sum_j e_j y_j[a] y_j[b] = (Y^T (e o Y))[a][b]   (e = 1, or -dvec)
// One CTA per (head, chunk).  A 128-token tile of y, as TMA delivers it, is at once the MN-major A
// operand (features along M) and -- when e = 1 -- the MN-major B operand; with e = -dvec four warps
// write the scaled rows e_j y_j (rounded to bf16 once, from the fp32 product) into a second tile
// with the same swizzled offsets.  An M = 128 operand has two 64-wide blocks; the second one is
// simply the 16 KB that follow the tile in shared memory (the next ring stage, or the first scaled
// tile after the last stage), so TMEM lanes 64..127 receive products of whatever lies there and are
// never read; lane a < 64, column b of the accumulator is E[a][b].  The result is left as a dense
// 64 x 64 block in the state matrix's own first-order rows (4096.. of 4161, 17.7 KB), which nothing has
// written yet: state_tc_kernel, next on the stream, copies E[a][b] into column 64 of the row (a, b) it
// writes anyway (4-byte stores scattered over 4096 rows cost more than the whole product), and the
// first-order state kernels then overwrite the block with the real rows.
constexpr int EC_THREADS = 192;       // warps 0-3: scaled copy and epilogue; 4: TMA; 5: MMA issuer
constexpr int EC_NS = 4;              // y-tile ring
constexpr int EC_STAGE = ST_ZTILE;
constexpr int EC_OFF_B = EC_NS * EC_STAGE;           // two scaled tiles
constexpr int EC_OFF_BAR = EC_OFF_B + 2 * ST_ZTILE;
constexpr int EC_NBAR = 2 * EC_NS + 4 + 1;
constexpr int EC_OFF_TMEM = EC_OFF_BAR + EC_NBAR * 8;
constexpr int EC_SMEM = EC_OFF_TMEM + 16 + 1024;

__global__ void __launch_bounds__(EC_THREADS, 2)
state_ecol_tc_kernel(const __grid_constant__ CUtensorMap tmY, const float* __restrict__ dvec,
                     float* __restrict__ state, int n, int chunk, int nchunk, int dvp, size_t per_state,
                     int skip_chunk) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + EC_OFF_BAR;
  // barriers: y_full[NS] | y_empty[NS] | b_full[2] | b_empty[2] | done
  auto BAR_YFULL = [&](int s) { return bar0 + 8u * s; };
  auto BAR_YEMPTY = [&](int s) { return bar0 + 8u * (EC_NS + s); };
  auto BAR_BFULL = [&](int b) { return bar0 + 8u * (2 * EC_NS + b); };
  auto BAR_BEMPTY = [&](int b) { return bar0 + 8u * (2 * EC_NS + 2 + b); };
  const uint32_t BAR_DONE = bar0 + 8u * (2 * EC_NS + 4);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + EC_OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hc = blockIdx.x, head = hc / nchunk, ck = hc % nchunk;
  if (ck == skip_chunk) return;
  const int t_begin = ck * chunk, t_end = min(n, t_begin + chunk);
  const int nblk = (t_end - t_begin + 127) / 128;
  const bool scaled = dvec != nullptr;

  if (tid == 0) {
    for (int s = 0; s < EC_NS; ++s) { mbar_init(BAR_YFULL(s), 1); mbar_init(BAR_YEMPTY(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(BAR_BFULL(b), 4); mbar_init(BAR_BEMPTY(b), 1); }
    mbar_init(BAR_DONE, 1);
    mbar_fence_init();
  }
  if (warp == 5) tmem_alloc(smem_u32((const void*)tmem_slot), 64);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) tma_prefetch_desc(&tmY);
    for (int k = 0; k < nblk; ++k) {
      const int s = k % EC_NS;
      if (!mbar_wait(BAR_YEMPTY(s), (((k / EC_NS) & 1) ^ 1))) { report(41); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_YFULL(s), EC_STAGE);
        // rows past the end of the sequence are zero-filled; chunks are whole multiples of 128 tokens
        tma_load_3d(sbase + s * EC_STAGE, &tmY, BAR_YFULL(s), 0, t_begin + k * 128, head);
      }
    }
  } else if (warp == 5) {
    constexpr uint32_t idesc = idesc_bf16(128, 64, 1, 1);
    bool ok = true;
    for (int k = 0; ok && k < nblk; ++k) {
      const int s = k % EC_NS, bb = k & 1;
      if (!mbar_wait_warp(BAR_YFULL(s), (uint32_t)((k / EC_NS) & 1))) { report(42); ok = false; break; }
      if (scaled && !mbar_wait_warp(BAR_BFULL(bb), (uint32_t)((k >> 1) & 1))) { report(43); ok = false; break; }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_lo = desc_lo(sbase + s * EC_STAGE, ST_ZTILE);
        const uint32_t b_lo = scaled ? desc_lo(sbase + EC_OFF_B + bb * ST_ZTILE, ST_ZTILE) : a_lo;
        umma_ss_mn_steps<8>(tmem, a_lo, b_lo, idesc, k > 0 ? 1u : 0u);
        umma_commit(BAR_YEMPTY(s));
        if (scaled) umma_commit(BAR_BEMPTY(bb));
      }
      __syncwarp();
    }
    if (ok && elect_one()) umma_commit(BAR_DONE);
    __syncwarp();
  } else {
    bool ok = true;
    if (scaled) {
      // thread j owns token row j of the block: the eight 16-byte pieces of the row keep their
      // (swizzled) offsets, so the copy never has to know which piece is which
      for (int k = 0; ok && k < nblk; ++k) {
        const int s = k % EC_NS, bb = k & 1;
        const int tok = t_begin + k * 128 + tid;
        const float e = (tok < t_end) ? -__ldg(dvec + (size_t)head * n + tok) : 0.f;
        if (!mbar_wait(BAR_YFULL(s), (uint32_t)((k / EC_NS) & 1))) { report(44); ok = false; break; }
        if (!mbar_wait(BAR_BEMPTY(bb), (uint32_t)(((k >> 1) & 1) ^ 1))) { report(45); ok = false; break; }
        const uint32_t src = sbase + s * EC_STAGE + tid * 128, dst = sbase + EC_OFF_B + bb * ST_ZTILE + tid * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 w = lds128(src + c * 16);
          const uint32_t in[4] = {w.x, w.y, w.z, w.w};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            o[q] = pack_bf16(e * __uint_as_float(in[q] << 16), e * __uint_as_float(in[q] & 0xFFFF0000u));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + c * 16), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                       "r"(o[3]) : "memory");
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_BFULL(bb));
      }
    }
    if (ok && !mbar_wait(BAR_DONE, 0)) { report(46); ok = false; }
    tc_fence_after();
    if (ok && warp < 2) {
      uint32_t tv[64];
      tmem_ld64(tmem + ((uint32_t)(warp * 32) << 16), tv);
      tmem_wait_ld();
      // E[a][0..63] as one contiguous row of the scratch block (see the header comment)
      float4* row = (float4*)(state + (size_t)hc * per_state + (size_t)4096 * dvp + (size_t)(warp * 32 + lane) * 64);
#pragma unroll
      for (int e = 0; e < 16; ++e)
        row[e] = make_float4(__uint_as_float(tv[4 * e]), __uint_as_float(tv[4 * e + 1]),
                             __uint_as_float(tv[4 * e + 2]), __uint_as_float(tv[4 * e + 3]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 64);
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                             CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeFn)p;
  }();
  return fn;
}
// (mats, rows, 64) bf16 as a rank-3 map with boxes of 128 x 64, 128-byte swizzle
int make_map(CUtensorMap* m, const void* base, size_t mats, size_t rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3] = {64, (cuuint64_t)rows, (cuuint64_t)mats};
  cuuint64_t gstr[2] = {128, (cuuint64_t)rows * 128};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return FASTMAX_OK;
}

}  // namespace

int moments_tc_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_mtc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}
int moments_tc_status_reset(cudaStream_t stream) {
  const int zero = 0;
  FM_CUDA_TRY(cudaMemcpyToSymbolAsync(g_mtc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}

// impl == FASTMAX_IMPL_MOMENTS_FFMA, or FASTMAX_B200_NO_TC_MOMENTS=1 in the environment, keeps the
// moment family on the CUDA-core kernels (used by the tests to compare the two implementations of
// the same stages).
bool moments_tc_supports(const fastmax_problem& p) {
  static const bool off = [] {
    const char* e = getenv("FASTMAX_B200_NO_TC_MOMENTS");
    return e && e[0] == '1';
  }();
  return !off && p.impl != FASTMAX_IMPL_MOMENTS_FFMA && p.dtype == FASTMAX_BF16 && p.d == 64 && p.p == 2 && p.bh == p.bhkv;
}

size_t moments_tc_state_bytes(int mats) { return (size_t)mats * NROWS_TP * 64 * 2; }

int moments_tc_convert(const Ctx& c, int mats, const float* state, void* state_bf16) {
  if (mats == 0) return FASTMAX_OK;
  const MomentDims m = moment_dims(64);
  dim3 grid(65, mats);
  FM_LAUNCH("fm_moments_state_bf16", c.stream,
            (state_to_bf16t_kernel<<<grid, 256, 0, c.stream>>>(state, (__nv_bfloat16*)state_bf16, m.dvp,
                                                               (size_t)m.f * m.dvp)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// Exclusive running sums over chunks (from `base`, per head, may be null) of the second-order rows,
// written as the read-out's bf16 transposed copies; the fp32 states stay raw.  The first-order rows
// are the caller's business (moments_prefix with a row range).
int moments_tc_prefix_convert(const Ctx& c, int heads, int nchunk, const float* state, const float* base,
                              int reverse, void* state_bf16) {
  if (heads == 0 || nchunk == 0) return FASTMAX_OK;
  const MomentDims m = moment_dims(64);
  if ((((uintptr_t)state | (uintptr_t)base) & 15) != 0)
    return fail(FASTMAX_E_ARG, "moment states and totals must be 16-byte aligned");
  dim3 grid(65, heads);
  FM_LAUNCH("fm_moments_prefix_bf16", c.stream,
            (prefix_bf16t_kernel<<<grid, 256, 0, c.stream>>>(state, base, (__nv_bfloat16*)state_bf16, nchunk,
                                                             m.dvp, (size_t)m.f * m.dvp, reverse)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// Second-order rows of the chunk states of (y, z | e) on the tensor cores: columns 0..63 by
// state_tc_kernel, the e column (e = 1 when dvec is null, else -dvec) by state_ecol_tc_kernel.
// The first-order and constant rows are NOT valid afterwards (they held the e column's scratch
// block): the caller builds them next, with first_tc_chunk_state or moments_chunk_state's p = 1
// row range, both of which write every element of those rows.
int moments_tc_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                           const float* dvec, float* state) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const MomentDims m = moment_dims(64);
  const int nchunk = (n + chunk - 1) / chunk;
  CUtensorMap tz;
  int rc;
  if ((rc = make_map(&tz, z, heads, n))) return rc;
  StArgs a;
  a.y = y; a.state = state; a.n = n; a.chunk = chunk; a.nchunk = nchunk; a.dvp = m.dvp;
  a.per_state = (size_t)m.f * m.dvp;
  a.skip_chunk = c.skip_chunk;
  // the normaliser column first: the state kernel picks it up in its epilogue
  CUtensorMap ty;
  if ((rc = make_map(&ty, y, heads, n))) return rc;
  FM_CUDA_TRY(cudaFuncSetAttribute(state_ecol_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, EC_SMEM));
  FM_LAUNCH("fm_moments_state_ecol", c.stream,
            (state_ecol_tc_kernel<<<(unsigned)((size_t)heads * nchunk), EC_THREADS, EC_SMEM, c.stream>>>(
                ty, dvec, state, n, chunk, nchunk, m.dvp, a.per_state, a.skip_chunk)));
  FM_CUDA_TRY(cudaGetLastError());
  FM_CUDA_TRY(cudaFuncSetAttribute(state_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM));
  FM_LAUNCH("fm_moments_tc_state", c.stream,
            (state_tc_kernel<<<(unsigned)((size_t)heads * nchunk * ST_SPLIT), ST_THREADS, ST_SMEM, c.stream>>>(tz, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// mode 0: type A on x -> out_a (+ den_a);  mode 1: type B on (x, u, uvec) -> out_b;
// mode 2: both on the same tokens.  Results overwrite; type B holds the second-order part only, type A the
// whole result when state_f32 (the fp32 states with summed first-order rows) is given.
int moments_tc_readout(const Ctx& c, int mode, int heads, int n, int chunk, int state_per_chunk,
                       const void* x, const void* u, const float* uvec, const void* state_bf16,
                       const stat_t* stats, float* out_a, float* den_a, float* out_b, const float* state_f32) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const fastmax_problem& p = c.p;
  const int nchunk = (n + chunk - 1) / chunk;
  CUtensorMap tx, ts, tu;
  int rc;
  const bool first_b = mode != 0 && state_f32 != nullptr && u != nullptr;
  if ((rc = make_map(&tx, x, heads, n))) return rc;
  if ((rc = make_map(&tu, first_b ? u : x, heads, n))) return rc;
  if ((rc = make_map(&ts, state_bf16, (size_t)heads * (state_per_chunk ? nchunk : 1), NROWS_TP))) return rc;
  RtArgs a;
  a.first_b = first_b ? 1 : 0;
  a.x = x; a.u = u; a.uvec = uvec; a.out_a = out_a; a.den_a = den_a; a.out_b = out_b;
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.a2 = p.a2; a.lim = p.lim;
  a.n = n; a.chunk = chunk; a.nchunk = nchunk; a.state_per_chunk = state_per_chunk; a.mode = mode;
  a.wide_io = (((uintptr_t)out_a | (uintptr_t)out_b) & 31) == 0;
  a.zero_chunk = state_per_chunk ? c.zero_chunk : -1;
  const MomentDims md = moment_dims(64);
  a.state_f32 = state_f32; a.per_state = (size_t)md.f * md.dvp; a.dvp = md.dvp; a.a0 = p.a0; a.a1 = p.a1;
  const int per_cta = (mode == 2) ? 128 : 256;
  const unsigned grid = (unsigned)((size_t)heads * ((n + per_cta - 1) / per_cta));
  FM_CUDA_TRY(cudaFuncSetAttribute(readout_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM));
  static const char* const names[3] = {"fm_moments_tc_readout_a", "fm_moments_tc_readout_b",
                                       "fm_moments_tc_readout_ab"};
  FM_LAUNCH(names[mode], c.stream, (readout_tc_kernel<<<grid, RT_THREADS, RT_SMEM, c.stream>>>(tx, ts, tu, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace fm
