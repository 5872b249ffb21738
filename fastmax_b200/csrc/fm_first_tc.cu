// First-order part of the moment-state form on the tcgen05 tensor cores (bf16 operands,
// fp32 accumulation), head dimension 64 or 128.  This is the whole computation when p = 1
// -- the case the reference's current CUDA kernels implement (fastmax_cuda_forward.cu:
// 25-197, fastmax_cuda_backward.cu:26-871: moments Sum v, Sum k, Sum k (x) v and their
// gradient counterparts) -- and the first-order rows of the state when p = 2.
//
//   state    S1[a][c] = sum_j y_j[a] z_j[c]          one MMA per 128-token tile: both operands
//                                                     are the raw token tiles TMA delivered
//                                                     (A = Y^T and B = Z, both MN-major)
//            S1[a][D] = sum_j y_j[a] e_j,  S0[c] = sum_j z_j[c],  S0[D] = sum_j e_j
//                                                     small vector sums on the CUDA cores
//   readout A  r_i[c] = A1 sum_a x_i[a] S1[a][c] + A0 S0[c]           (c <= D; c = D: normaliser)
//   readout B  r_i[a] = A1 (sum_c u_i[c] S1[a][c] + e_i S1[a][D])
//                                                     one GEMM of the raw token tile against a
//                                                     bf16 copy of S1 (MN-major B for type A,
//                                                     the same bytes K-major for type B)
// All of it is bound by HBM traffic: every token row is read once per stage.
#include <cstdlib>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_ftc_status = 0;  // first protocol error seen by a kernel of this file

namespace {
using namespace sm100;

__device__ __forceinline__ void report(int code) { atomicCAS(&g_ftc_status, 0, code); }

constexpr int F1_THREADS = 192;  // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: vector sums, epilogue

// =====================================================================================
// state build
// =====================================================================================
struct F1StateArgs {
  const void* y;       // (heads, n, D) bf16 feature source (k, or q)
  const void* z;       // (heads, n, D) bf16 values (v, or grad_out/den)
  const float* dvec;   // e_j = -dvec[j] when not null, else 1
  float* state;        // (heads, nchunk, rows, DVP) fp32; rows f_lin .. f_lin + D are written
  int n, chunk, nchunk, dvp, rows, f_lin;   // f_lin: stored index of the first first-order row
  int skip_chunk;      // this chunk's state is not wanted (-1: none)
};

template <int DD>
struct F1S {
  static constexpr int NSUB = DD / 64;
  // Tokens per tile and ring depth are chosen so that a CTA needs 96 KB of shared memory: two CTAs per SM,
  // each with two of its three 32 KB stages in flight while the third is consumed, keep enough bytes on the
  // way from HBM (one CTA with two 64 KB stages reached 58 % of the copy bandwidth).
  static constexpr int TOK = (DD == 128) ? 64 : 128;
  static constexpr int NS = 3;
  static constexpr int SUBTILE = TOK * 128;       // TOK tokens x 64 bf16
  static constexpr int TILE = NSUB * SUBTILE;     // one operand tile: TOK tokens x DD bf16
  static constexpr int STAGE = 2 * TILE;          // Y then Z
  static constexpr int OFF_VEC = NS * STAGE;      // float sv[DD], se[DD], s_e, pad, e[128]
  static constexpr int OFF_BAR = OFF_VEC + (2 * DD + 4 + 128) * 4;
  static constexpr int NBAR = 2 * NS + 1;
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;
};

template <int DD>
__global__ void __launch_bounds__(F1_THREADS, 2)
first_state_kernel(const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmZ,
                   const F1StateArgs a) {
  using C = F1S<DD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR_FULL = [&](int s) { return bar0 + 8u * s; };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (C::NS + s); };
  auto BAR_DONE = [&]() { return bar0 + 8u * (2 * C::NS); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + C::OFF_TMEM);
  float* vsum = (float*)(smem + C::OFF_VEC);      // [0,DD): sum z, [DD,2DD): sum y e, [2DD]: sum e

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hc = blockIdx.x, head = hc / a.nchunk, chunk = hc % a.nchunk;
  if (chunk == a.skip_chunk) return;
  const int t_begin = chunk * a.chunk, t_end = min(a.n, t_begin + a.chunk);
  constexpr int TOK = C::TOK;
  const int nblk = (t_end - t_begin + TOK - 1) / TOK;

  if (tid == 0) {
    // a stage is free when the MMAs that read it are done and the vector sums have read it
    for (int s = 0; s < C::NS; ++s) { mbar_init(BAR_FULL(s), 1); mbar_init(BAR_EMPTY(s), 2); }
    mbar_init(BAR_DONE(), 1);
    mbar_fence_init();
  }
  for (int i = tid; i < 2 * DD + 4; i += F1_THREADS) vsum[i] = 0.f;
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) { tma_prefetch_desc(&tmY); tma_prefetch_desc(&tmZ); }
    for (int k = 0; k < nblk; ++k) {
      const int s = k % C::NS;
      if (!mbar_wait(BAR_EMPTY(s), (((k / C::NS) & 1) ^ 1))) { report(41); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), C::STAGE);
        const uint32_t dst = sbase + s * C::STAGE;
        for (int sub = 0; sub < C::NSUB; ++sub) {
          tma_load_3d(dst + sub * C::SUBTILE, &tmY, BAR_FULL(s), sub * 64, t_begin + k * TOK, head);
          tma_load_3d(dst + C::TILE + sub * C::SUBTILE, &tmZ, BAR_FULL(s), sub * 64, t_begin + k * TOK, head);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // M = 128 rows of the accumulator; with DD = 64 the second 64-row block of A is the Z
      // tile that follows Y in the stage (valid memory), and those rows are never read back
      constexpr uint32_t idesc = idesc_bf16(128, DD, 1, 1);
      bool ok = true;
      for (int k = 0; ok && k < nblk; ++k) {
        const int s = k % C::NS;
        if (!mbar_wait(BAR_FULL(s), (uint32_t)((k / C::NS) & 1))) { report(42); ok = false; break; }
        tc_fence_after();
        const uint32_t y_lo = desc_lo(sbase + s * C::STAGE, C::SUBTILE);
        const uint32_t z_lo = desc_lo(sbase + s * C::STAGE + C::TILE, C::SUBTILE);
        umma_ss_mn_steps<TOK / 16>(tmem, y_lo, z_lo, idesc, k > 0 ? 1u : 0u);
        umma_commit(BAR_EMPTY(s));
      }
      if (ok) umma_commit(BAR_DONE());
    }
    __syncwarp();
  } else {
    // ---- vector sums over the chunk's tokens, read from the tiles TMA delivered ----
    // element (row r, column c) of a 64-column sub-tile sits at r*128 + (((c>>3) ^ (r&7))<<4) + (c&7)*2
    const int t = tid - 64;                       // 0..127
    constexpr int HP = DD / 2;                    // bf16 pairs per row
    constexpr int NPART = 128 / HP;               // threads per column pair, interleaved over rows
    const int cp = t % HP, part = t / HP;
    const int sub = (2 * cp) >> 6, cc = (2 * cp) & 63;
    const float* dv = a.dvec ? a.dvec + (size_t)head * a.n : nullptr;
    float* ebuf = vsum + 2 * DD + 4;
    float2 sz = make_float2(0.f, 0.f), sye = sz;
    float se = 0.f;
    bool ok = true;
    for (int k = 0; k < nblk; ++k) {
      const int s = k % C::NS;
      const int tok0 = t_begin + k * TOK;
      if (t < TOK) ebuf[t] = (tok0 + t < t_end) ? (dv ? -__ldg(dv + tok0 + t) : 1.f) : 0.f;
      if (!mbar_wait(BAR_FULL(s), (uint32_t)((k / C::NS) & 1))) { report(46); ok = false; break; }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint8_t* yt = smem + s * C::STAGE + sub * C::SUBTILE;
      const uint8_t* zt = yt + C::TILE;
#pragma unroll 4
      for (int r = part; r < TOK; r += NPART) {
        const uint32_t off = r * 128 + ((((uint32_t)cc >> 3) ^ (r & 7)) << 4) + (cc & 7) * 2;
        const float e = ebuf[r];                  // 0 for rows past the end of the chunk
        const float2 zv = __bfloat1622float2(*(const __nv_bfloat162*)(zt + off));
        const float2 yv = __bfloat1622float2(*(const __nv_bfloat162*)(yt + off));
        if (tok0 + r < t_end) { sz.x += zv.x; sz.y += zv.y; }
        sye.x = fmaf(yv.x, e, sye.x); sye.y = fmaf(yv.y, e, sye.y);
        se += e;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (t == 0) mbar_arrive(BAR_EMPTY(s));
    }
    atomicAdd(&vsum[2 * cp], sz.x);
    atomicAdd(&vsum[2 * cp + 1], sz.y);
    atomicAdd(&vsum[DD + 2 * cp], sye.x);
    atomicAdd(&vsum[DD + 2 * cp + 1], sye.y);
    if (cp == 0) atomicAdd(&vsum[2 * DD], se);
    // named barrier among the four epilogue warps only
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // ---- epilogue ----
    if (ok && !mbar_wait(BAR_DONE(), 0)) { report(43); ok = false; }
    tc_fence_after();
    float* st = a.state + (size_t)hc * a.rows * a.dvp;
    const int qd = warp & 3;                      // TMEM lane quarter this warp may read
    if (ok && qd * 32 < DD) {
      const int arow = qd * 32 + lane;            // accumulator row = feature index a
      float* dst = st + (size_t)(a.f_lin + arow) * a.dvp;
#pragma unroll 1
      for (int hcol = 0; hcol < DD / 64; ++hcol) {
        uint32_t tv[64];
        tmem_ld64(tmem + ((uint32_t)(qd * 32) << 16) + hcol * 64, tv);
        tmem_wait_ld();
#pragma unroll
        for (int e4 = 0; e4 < 16; ++e4)
          ((float4*)(dst + hcol * 64))[e4] = make_float4(__uint_as_float(tv[4 * e4]), __uint_as_float(tv[4 * e4 + 1]),
                                                         __uint_as_float(tv[4 * e4 + 2]), __uint_as_float(tv[4 * e4 + 3]));
      }
      dst[DD] = vsum[DD + arow];
      for (int cc = DD + 1; cc < a.dvp; ++cc) dst[cc] = 0.f;
    }
    // constant row: [sum z | sum e | 0]
    float* crow = st + (size_t)(a.f_lin + DD) * a.dvp;
    for (int cc = t; cc < a.dvp; cc += 128) crow[cc] = (cc < DD) ? vsum[cc] : (cc == DD ? vsum[2 * DD] : 0.f);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}


// =====================================================================================
// read-out
// =====================================================================================
struct F1ReadArgs {
  const void* x;        // (heads, n, D) bf16 tokens (type A: the MMA operand; both: normaliser dot)
  const float* uvec;    // type B: e_i = -uvec[i] when not null, else 1
  const float* state;   // fp32 states (first-order rows are read for the vector terms)
  float* o_add;         // (heads, n, D) fp32 result
  float* den_add;       // type A: (heads, n) normaliser part, may be null
  const stat_t* stat_q;
  const stat_t* stat_k;
  float a0, a1, lim;
  int n, chunk, nchunk, per_chunk, dvp, rows, f_lin, type_b, accumulate;
  int run;              // tiles per CTA (all of one state)
  // final != 0: the read-out is the whole result (p = 1, unmasked): write bf16 rows to out_final
  // instead of fp32 to o_add.  1: type A divided by its normaliser (which goes to den_final);
  // 2: plain rounding; the per-head dot with x is added to *dots when dots is not null.
  int final;
  void* out_final;
  float* den_final;
  float* dots;
  int wide_io;          // out_final / o_add / x are 32-byte aligned: 32-byte accesses in the epilogue
  int zero_chunk;       // per-chunk mode: the tokens of this chunk read an empty state (-1: none)
};

// 16 bytes from shared memory by shared-window address (keeps the epilogue's vector reads off the generic path)
__device__ __forceinline__ uint4 lds128u(uint32_t saddr) {
  uint4 r;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(saddr));
  return r;
}
__device__ __forceinline__ float4 lds128f(uint32_t saddr) {
  float4 r;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(saddr));
  return r;
}

template <int DD>
struct F1R {
  static constexpr int NSUB = DD / 64;
  static constexpr int TILE = NSUB * 16384;        // 128 tokens x DD bf16
  static constexpr int SMAT = DD * DD * 2;         // bf16 copy of S1, NSUB sub-tiles of DD rows x 64
  static constexpr int OFF_S = 2 * TILE;           // two token-tile stages first
  static constexpr int OFF_VEC = OFF_S + SMAT;     // normaliser column [DD] | constant row [DD + 1]
  static constexpr int OFF_BAR = OFF_VEC + (2 * DD + 8) * 4;
  static constexpr int NBAR = 9;                   // s_full | t_full[2] | t_empty[2] | a_full[2] | a_free[2]
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;
  static constexpr int TCOLS = 2 * DD;             // two accumulators
};

// One CTA reads out a run of consecutive 128-token tiles that share one state: the bf16 state
// copy is loaded once, token tiles stream through two stages, and two TMEM accumulators let the
// epilogue of a tile overlap the load and the product of the next one.
template <int DD>
__global__ void __launch_bounds__(F1_THREADS, 2)
first_readout_kernel(const __grid_constant__ CUtensorMap tmT, const __grid_constant__ CUtensorMap tmS,
                     const F1ReadArgs a) {
  using C = F1R<DD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  const uint32_t BAR_SF = bar0;
  auto BAR_TF = [&](int b) { return bar0 + 8u * (1 + b); };
  auto BAR_TE = [&](int b) { return bar0 + 8u * (3 + b); };
  auto BAR_AF = [&](int b) { return bar0 + 8u * (5 + b); };
  auto BAR_AE = [&](int b) { return bar0 + 8u * (7 + b); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + C::OFF_TMEM);
  float* ncol = (float*)(smem + C::OFF_VEC);       // S1[a][DD], a < DD
  float* crow = ncol + DD;                         // constant row, DD + 1 values
  const uint32_t ncol_s = sbase + C::OFF_VEC;      // the same vectors by shared-window address
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles = (a.n + 127) / 128;
  const int runs = (tiles + a.run - 1) / a.run;
  const int head = blockIdx.x / runs;
  const int tile0 = (blockIdx.x % runs) * a.run;
  const int nt = min(a.run, tiles - tile0);        // tiles of this run
  const int mat = head * (a.per_chunk ? a.nchunk : 1) + (a.per_chunk ? (tile0 * 128) / a.chunk : 0);
  if (a.per_chunk && (tile0 * 128) / a.chunk == a.zero_chunk) {
    // the run lies in one chunk, whose state is empty: the result is zero -- nothing to add, or zeros to write
    if (!a.accumulate) {
      const int row0 = tile0 * 128, rows = min(nt * 128, a.n - row0);
      for (int i = tid; i < rows * (DD / 4); i += F1_THREADS)
        *(float4*)(a.o_add + ((size_t)head * a.n + row0) * DD + (size_t)i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!a.type_b && a.den_add)
        for (int i = tid; i < rows; i += F1_THREADS) a.den_add[(size_t)head * a.n + row0 + i] = 0.f;
    }
    return;
  }

  if (tid == 0) {
    mbar_init(BAR_SF, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(BAR_TF(b), 1);
      // a stage is free once the product that read it is done and, where the epilogue reads x from it for
      // the normaliser dot (type A), once its four warps have done so
      mbar_init(BAR_TE(b), (!a.type_b && (a.den_add || a.final == 1)) ? 5 : 1);
      mbar_init(BAR_AF(b), 1);
      mbar_init(BAR_AE(b), 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), C::TCOLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      mbar_expect_tx(BAR_SF, C::SMAT);
      for (int sub = 0; sub < C::NSUB; ++sub)
        tma_load_3d(sbase + C::OFF_S + sub * (DD * 128), &tmS, BAR_SF, sub * 64, 0, mat);
    }
    for (int i = 0; i < nt; ++i) {
      const int b = i & 1;
      if (!mbar_wait(BAR_TE(b), (uint32_t)(((i >> 1) & 1) ^ 1))) { report(47); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_TF(b), C::TILE);
        for (int sub = 0; sub < C::NSUB; ++sub)
          tma_load_3d(sbase + b * C::TILE + sub * 16384, &tmT, BAR_TF(b), sub * 64, (tile0 + i) * 128, head);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (whole warp, one elected lane issues) =================
    bool ok = mbar_wait_warp(BAR_SF, 0);
    if (!ok) report(44);
    for (int i = 0; ok && i < nt; ++i) {
      const int b = i & 1;
      if (!mbar_wait_warp(BAR_TF(b), (uint32_t)((i >> 1) & 1))) { report(44); break; }
      if (!mbar_wait_warp(BAR_AE(b), (uint32_t)(((i >> 1) & 1) ^ 1))) { report(48); break; }
      tc_fence_after();
      const uint32_t t_lo = desc_lo(sbase + b * C::TILE, 16);
      const uint32_t acc = tmem + b * DD;
      if (elect_one()) {
        if (a.type_b) {
          // acc[i][a'] = sum_c u_i[c] S1[a'][c]: B = S1 rows a' with c contiguous (K-major)
          constexpr uint32_t idesc = idesc_bf16(128, DD, 0, 0);
          const uint32_t s_lo = desc_lo(sbase + C::OFF_S, 16);
#pragma unroll
          for (int sub = 0; sub < C::NSUB; ++sub)
            umma_ss_k64(acc, t_lo + sub * (16384 >> 4), s_lo + sub * ((DD * 128) >> 4), idesc, sub > 0);
        } else {
          // acc[i][c] = sum_a x_i[a] S1[a][c]: B = the same bytes, K = rows a, N = c contiguous (MN-major)
          constexpr uint32_t idesc = idesc_bf16(128, DD, 0, 1);
          const uint32_t s_lo = desc_lo(sbase + C::OFF_S, DD * 128);
#pragma unroll
          for (int sub = 0; sub < C::NSUB; ++sub)
            umma_ss_kmn_steps<4>(acc, t_lo + sub * (16384 >> 4), s_lo + sub * 4 * 128, idesc, sub > 0);
        }
        umma_commit(BAR_AF(b));
        umma_commit(BAR_TE(b));
      }
      __syncwarp();
    }
    __syncwarp();
  } else {
    // ================= epilogue warps =================
    const int qd = warp & 3, t = tid - 64;
    const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head, a.lim);
    const float A1 = a.a1 * c;
    const float* st = a.state + (size_t)mat * a.rows * a.dvp + (size_t)a.f_lin * a.dvp;   // first-order rows
    for (int i = t; i < 2 * DD + 1; i += 128)
      ncol[i] = (i < DD) ? __ldg(st + (size_t)i * a.dvp + DD) : __ldg(st + (size_t)DD * a.dvp + (i - DD));
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // type A adds a0 * (constant row) to every element: scaled once here (the value column DD stays raw);
    // the loops below read these vectors four values per shared-memory access
    if (!a.type_b)
      for (int i = t; i < DD; i += 128) crow[i] *= a.a0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    float part = 0.f;
    bool ok = true;
    for (int i = 0; i < nt; ++i) {
      const int b = i & 1;
      const int tok = (tile0 + i) * 128 + qd * 32 + lane;
      const bool tok_ok = tok < a.n;
      const size_t grow = (size_t)head * a.n + (tok_ok ? tok : 0);
      float extra = 0.f;   // type A: normaliser part; type B: e_i
      if (a.type_b) {
        extra = tok_ok ? (a.uvec ? -a.uvec[grow] : 1.f) : 0.f;
      } else if (a.den_add || a.final == 1) {
        // x_i . (normaliser column): the row is read from the token tile TMA delivered (128-byte rows of a
        // 64-column sub-tile, 16-byte pieces XOR-swizzled by the row), not from global memory again
        if (!mbar_wait(BAR_TF(b), (uint32_t)((i >> 1) & 1))) { report(49); ok = false; break; }
        const int r = qd * 32 + lane;
        const uint32_t trow = sbase + b * C::TILE + r * 128;
        float dot = 0.f;
#pragma unroll
        for (int sb = 0; sb < C::NSUB; ++sb)
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) {
            const uint4 xv = lds128u(trow + sb * 16384 + ((pc ^ (r & 7)) << 4));
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
            const float4 n0 = lds128f(ncol_s + (sb * 64 + 8 * pc) * 4), n1 = lds128f(ncol_s + (sb * 64 + 8 * pc + 4) * 4);
            const float nc[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              dot = fmaf(__uint_as_float(xw[e] << 16), nc[2 * e], dot);
              dot = fmaf(__uint_as_float(xw[e] & 0xFFFF0000u), nc[2 * e + 1], dot);
            }
          }
        extra = A1 * dot + a.a0 * crow[DD];
        // this warp is done with the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_TE(b));
      }
      if (!mbar_wait(BAR_AF(b), (uint32_t)((i >> 1) & 1))) { report(45); ok = false; break; }
      tc_fence_after();
      const float scale = (a.final == 1) ? 1.0f / extra : 1.0f;
#pragma unroll 1
      for (int hcol = 0; hcol < DD / 64; ++hcol) {
        uint32_t tv[64];
        tmem_ld64(tmem + b * DD + ((uint32_t)(qd * 32) << 16) + hcol * 64, tv);
        tmem_wait_ld();
        if (hcol + 1 == DD / 64) {   // the accumulator is in registers: the next product may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_AE(b));
        }
        if (tok_ok) {
          const bool wide = a.wide_io != 0;
#pragma unroll
          for (int v16 = 0; v16 < 4; ++v16) {
            float r[16];
            const uint32_t vecp = (a.type_b ? ncol_s : ncol_s + DD * 4) + (hcol * 64 + 16 * v16) * 4;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const float4 c4 = lds128f(vecp + 16 * q4);
              const float cv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float acc = __uint_as_float(tv[16 * v16 + 4 * q4 + e]);
                r[4 * q4 + e] = a.type_b ? A1 * fmaf(extra, cv[e], acc) : fmaf(A1, acc, cv[e]);
              }
            }
            if (a.final) {
              uint32_t w[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) w[e] = pack_bf16(r[2 * e] * scale, r[2 * e + 1] * scale);
              stg32((__nv_bfloat16*)a.out_final + grow * DD + hcol * 64 + 16 * v16, w, wide);
              if (a.dots) {
                uint32_t xw[8];
                ldg32((const __nv_bfloat16*)a.x + grow * DD + hcol * 64 + 16 * v16, xw, wide);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  part = fmaf(r[2 * e], __uint_as_float(xw[e] << 16), part);
                  part = fmaf(r[2 * e + 1], __uint_as_float(xw[e] & 0xFFFF0000u), part);
                }
              }
            } else {
#pragma unroll
              for (int h8 = 0; h8 < 2; ++h8) {
                float* dst = a.o_add + grow * DD + hcol * 64 + 16 * v16 + 8 * h8;
                uint32_t w[8];
                if (a.accumulate) {
                  ldg32(dst, w, wide);
#pragma unroll
                  for (int e = 0; e < 8; ++e) w[e] = __float_as_uint(r[8 * h8 + e] + __uint_as_float(w[e]));
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) w[e] = __float_as_uint(r[8 * h8 + e]);
                }
                stg32(dst, w, wide);
              }
            }
          }
        }
      }
      if (a.final) {
        if (a.final == 1 && tok_ok) a.den_final[grow] = extra;
      } else if (!a.type_b && a.den_add && tok_ok) {
        a.den_add[grow] = extra + (a.accumulate ? a.den_add[grow] : 0.f);
      }
    }
    if (ok && a.final && a.dots) {
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
      if (lane == 0) atomicAdd(a.dots + head, part);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TCOLS);
  }
}

// bf16 copy of the first-order block: out[m][a][c] = state[m][f_lin + a][c], a, c < D
__global__ void __launch_bounds__(256) s1_to_bf16_kernel(const float* __restrict__ state,
                                                         __nv_bfloat16* __restrict__ out, int d, int dvp,
                                                         int rows, int f_lin) {
  const float* src = state + (size_t)blockIdx.x * rows * dvp + (size_t)f_lin * dvp;
  __nv_bfloat16* dst = out + (size_t)blockIdx.x * d * d;
  for (int i = threadIdx.x; i < d * d; i += 256) dst[i] = __float2bfloat16_rn(src[(size_t)(i / d) * dvp + i % d]);
}

}  // namespace

// ---- host side ---------------------------------------------------------------------------
// FASTMAX_B200_NO_TC_MOMENTS=1 keeps the moment family on the CUDA-core kernels (see fm_moments_tc.cu).
bool first_tc_supports(const fastmax_problem& p) {
  static const bool off = [] {
    const char* e = getenv("FASTMAX_B200_NO_TC_MOMENTS");
    return e && e[0] == '1';
  }();
  return !off && p.impl != FASTMAX_IMPL_MOMENTS_FFMA && p.dtype == FASTMAX_BF16 && (p.d == 64 || p.d == 128) && p.bh == p.bhkv;
}

size_t first_tc_copy_bytes(const fastmax_problem& p, int mats) { return (size_t)mats * p.d * p.d * 2; }

int first_tc_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_ftc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}
int first_tc_status_reset(cudaStream_t stream) {
  const int zero = 0;
  FM_CUDA_TRY(cudaMemcpyToSymbolAsync(g_ftc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}

// First-order and constant rows of the chunk states of (y, z | e); e = 1 when dvec is null, else -dvec.
int first_tc_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                         const float* dvec, float* state) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const fastmax_problem& p = c.p;
  const MomentDims m = moment_dims(p.d, p.p);
  const int nchunk = (n + chunk - 1) / chunk;
  CUtensorMap ty, tz;
  int rc;
  const int tok = p.d == 128 ? F1S<128>::TOK : F1S<64>::TOK;
  if ((rc = tma_map_bf16(&ty, y, heads, n, p.d, tok))) return rc;
  if ((rc = tma_map_bf16(&tz, z, heads, n, p.d, tok))) return rc;
  F1StateArgs a;
  a.y = y; a.z = z; a.dvec = dvec; a.state = state;
  a.n = n; a.chunk = chunk; a.nchunk = nchunk; a.dvp = m.dvp; a.rows = m.f; a.f_lin = p.d * p.d - m.f0;
  a.skip_chunk = c.skip_chunk;
  const unsigned grid = (unsigned)((size_t)heads * nchunk);
  if (p.d == 128) {
    FM_CUDA_TRY(cudaFuncSetAttribute(first_state_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, F1S<128>::SMEM));
    FM_LAUNCH("fm_first_tc_state", c.stream, (first_state_kernel<128><<<grid, F1_THREADS, F1S<128>::SMEM, c.stream>>>(ty, tz, a)));
  } else {
    FM_CUDA_TRY(cudaFuncSetAttribute(first_state_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, F1S<64>::SMEM));
    FM_LAUNCH("fm_first_tc_state", c.stream, (first_state_kernel<64><<<grid, F1_THREADS, F1S<64>::SMEM, c.stream>>>(ty, tz, a)));
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// bf16 copies of the first-order blocks of `mats` prefix (or total) states
int first_tc_convert(const Ctx& c, int mats, const float* state, void* s1b) {
  if (mats == 0) return FASTMAX_OK;
  const fastmax_problem& p = c.p;
  const MomentDims m = moment_dims(p.d, p.p);
  FM_LAUNCH("fm_first_state_bf16", c.stream,
            (s1_to_bf16_kernel<<<mats, 256, 0, c.stream>>>(state, (__nv_bfloat16*)s1b, p.d, m.dvp, m.f,
                                                           p.d * p.d - m.f0)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// type A (type_b = 0): tile = x;  type B: tile = u (gs or v), uvec = dvec or null.  x is the token
// tensor itself (normaliser dot of type A).  Results overwrite o_add / den_add unless accumulate.
int first_tc_readout(const Ctx& c, int type_b, int heads, int n, int chunk, int per_chunk, const void* tile,
                     const void* x, const float* uvec, const float* state, const void* s1b,
                     const stat_t* stats, float* o_add, float* den_add, int accumulate, int final,
                     void* out_final, float* den_final, float* dots) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const fastmax_problem& p = c.p;
  const MomentDims m = moment_dims(p.d, p.p);
  const int nchunk = (n + chunk - 1) / chunk;
  CUtensorMap tt, ts;
  int rc;
  if ((rc = tma_map_bf16(&tt, tile, heads, n, p.d, 128))) return rc;
  if ((rc = tma_map_bf16(&ts, s1b, (size_t)heads * (per_chunk ? nchunk : 1), p.d, p.d, p.d))) return rc;
  F1ReadArgs a;
  a.x = x; a.uvec = uvec; a.state = state; a.o_add = o_add; a.den_add = den_add;
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.a0 = p.a0; a.a1 = p.a1; a.lim = p.lim;
  a.n = n; a.chunk = chunk; a.nchunk = nchunk; a.per_chunk = per_chunk; a.dvp = m.dvp; a.rows = m.f;
  a.f_lin = p.d * p.d - m.f0; a.type_b = type_b; a.accumulate = accumulate;
  a.final = final; a.out_final = out_final; a.den_final = den_final; a.dots = dots;
  a.wide_io = (((uintptr_t)out_final | (uintptr_t)o_add | (uintptr_t)x) & 31) == 0;
  a.zero_chunk = (per_chunk && !final) ? c.zero_chunk : -1;
  // runs of up to 8 tiles that never cross a chunk (chunks are multiples of 256 tokens)
  // a CTA pays for loading the state copy and the vector terms once per run, so runs are as long as
  // the chunk allows (a run never crosses a chunk; chunks are multiples of 256 tokens), at most 32 tiles --
  // shortened while that would leave the GPU short of CTAs
  const int tiles = (n + 127) / 128;
  int run = 32;
  if (per_chunk) {
    const int tpc = chunk / 128;
    while (tpc % run) run >>= 1;
  }
  while (run > 8 && (size_t)heads * ((tiles + run - 1) / run) < 4 * 148) run >>= 1;
  a.run = run;
  const unsigned grid = (unsigned)((size_t)heads * ((tiles + run - 1) / run));
  const char* name = type_b ? "fm_first_tc_readout_b" : "fm_first_tc_readout_a";
  if (p.d == 128) {
    FM_CUDA_TRY(cudaFuncSetAttribute(first_readout_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, F1R<128>::SMEM));
    FM_LAUNCH(name, c.stream, (first_readout_kernel<128><<<grid, F1_THREADS, F1R<128>::SMEM, c.stream>>>(tt, ts, a)));
  } else {
    FM_CUDA_TRY(cudaFuncSetAttribute(first_readout_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, F1R<64>::SMEM));
    FM_LAUNCH(name, c.stream, (first_readout_kernel<64><<<grid, F1_THREADS, F1R<64>::SMEM, c.stream>>>(tt, ts, a)));
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace fm
