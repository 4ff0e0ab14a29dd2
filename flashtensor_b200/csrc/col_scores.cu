// Per-key column reductions of the attention probabilities for sm_100a.
//
// Replaces the column kernel the Asuka pipeline generates beside the forward kernel for
//   h2o_score   = probs.sum(dim=2)                       (cases/kernels/h2o.py:35-36)
//   roco_score, roco_sq_score = sum p, sum p^2           (cases/kernels/roco.py:42-46)
//   kf_score    = softmax((scores + g)/tau).sum(dim=2)   (cases/kernels/kf.py:36-40)
// It needs every row's softmax denominator first, so it recomputes S from Q and K and reads the
// per-row base-2 log-sum-exp written by the forward kernel (or by the Keyformer row pass below).
//
// Orientation is transposed: S^T = K Q^T, so TMEM lane = key and one thread owns one key.  A
// key's sum over all query rows is then a serial f32 sum in one thread, in a fixed order: no
// cross-thread or cross-CTA reduction exists, and results are bitwise reproducible.
//   warp 0      producer: two resident K tiles (256 keys), Q tiles + their row statistics in a ring
//   warp 1      tcgen05.mma issuer: S^T_t[buf] = K_t Q_i^T into one of two TMEM buffers per key tile
//   warps 4-11  keys   0..127 of the block: exp2, mask, accumulate; two warps per 32 keys, one for
//               queries 0..63 and one for queries 64..127 of every query tile
//   warps 12-19 keys 128..255, likewise
// Four key warps per scheduler, not two: one warp's stream of FFMA -> MUFU -> FADD chains stalls
// on its own latencies about half the time, and its loads and barrier waits stall it outright, so
// two warps leave the MUFU idle a third of the time.
//
// The Keyformer row pass (kf_rowstat) is the row-oriented counterpart: S = Q K^T, one thread per
// query row, online max/sum of the perturbed logits, nothing else.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "../../include/asuka_b200.h"
#include "kernels.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace asuka {
using namespace sm100;

namespace {

constexpr int kTile = 128;
constexpr uint32_t kTileBytes = 128 * 128 * 2;
constexpr uint32_t kHalfBytes = kTileBytes / 2;
constexpr int kQStages = 4;
#ifndef ASUKA_COL_UTIL_WARPS
#define ASUKA_COL_UTIL_WARPS 2
#endif
constexpr int kUtilWarps = ASUKA_COL_UTIL_WARPS;  // producer and MMA issuer (no idle warps: their registers go to the key warps)
constexpr int kThreads = (kUtilWarps + 16) * 32;  // + 16 key warps; 576 threads x 112 registers, no setmaxnreg
constexpr uint32_t kSmemBytes = (2 + kQStages) * kTileBytes + 1024;

struct ColParams {
  int B, H, Sq, Skv;
  int causal, diag_off;
  int nq_tiles;
  int group;          // query heads per key head (grouped-query attention)
  float scale_log2;   // softmax_scale * log2(e) (perturbed mode: additionally / tau)
  float inv_tau;
  const float* lse2;  // [B,H,Sq]
  float* score;       // [B,H,Skv]
  float* score_sq;
  const float* exp_rand;
  int64_t er_sb, er_sh, er_sq;
  uint64_t seed;
  uint32_t unit_off;  // added to the (batch * H + head) index the seeded noise is keyed by
  uint32_t* status;
  int chained;        // the kernel ahead in the stream does not write q or k
  // Query-range split, for launches with too few key blocks to fill the SMs: the query tiles are
  // cut into `n_qchunks` ranges of `q_chunk` tiles, one CTA per (key block, range); every CTA
  // leaves its partial sums in `part` ([n_qchunks, B*H, Skv], and `part_sq` alike) and
  // sum_chunks_kernel adds them in range order.  n_qchunks = 1: no split, results go to `score`.
  int q_chunk, n_qchunks;
  float* part;
  float* part_sq;
};

struct ColBars {
  uint64_t k_full;
  uint64_t q_full[kQStages], q_empty[kQStages];
  uint64_t s_full[2][2], s_empty[2][2];
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// exp2 on the FMA pipe, two logits per instruction (packed f32x2): x = n + f with n = rint(x) taken
// from the mantissa of x + 1.5 * 2^23, a degree-4 polynomial for 2^f on [-0.5, 0.5] (relative
// error 2.7e-6), and n added into the exponent field.  The MUFU does 16 exponentials per clock per
// SM and is what bounds this kernel; giving a share of every tile's logits to the FMA pipe (128
// lanes per clock) lets both pipes run side by side.  The share is small: each such logit costs
// about 7 clocks of the FMA pipe per warp (packed instructions occupy it for two) against 8 of the
// MUFU, and the pipe also carries the scaling and the accumulation of every logit.  Inputs below -120 give 2^-120 (the column
// sums do not notice); inputs above 0 only occur at masked positions, which are zeroed afterwards.
#ifndef ASUKA_COL_POLY_QUARTERS
#define ASUKA_COL_POLY_QUARTERS 1  // of every four logits, how many go to the FMA pipe (0, 1, 2 or 3);
                                   // measured at S = 4096, 32 heads: 0 -> 96.9, 1 -> 91.3, 2 -> 92.7 us
#endif
#ifndef ASUKA_COL_POLY_DEG
#define ASUKA_COL_POLY_DEG 4
#endif
#ifndef ASUKA_COL_POLY_SCALAR
#define ASUKA_COL_POLY_SCALAR 0
#endif
__device__ __forceinline__ float ex2_fma_pipe1(float x) {
#ifndef ASUKA_COL_POLY_NOCLAMP
  x = fmaxf(x, -120.f);
#endif
  const float t = __fadd_rn(x, 12582912.f);
  const float n = __fadd_rn(t, -12582912.f);
  const float f = __fadd_rn(x, -n);
#if ASUKA_COL_POLY_DEG == 3
  float p = 0.055171605199575424f;
  p = __fmaf_rn(p, f, 0.2426111102104187f);
  p = __fmaf_rn(p, f, 0.6932609677314758f);
  p = __fmaf_rn(p, f, 0.9999280571937561f);
#else
  float p = 0.009570094756782055f;
  p = __fmaf_rn(p, f, 0.05591785907745361f);
  p = __fmaf_rn(p, f, 0.240247443318367f);
  p = __fmaf_rn(p, f, 0.6931217908859253f);
  p = __fmaf_rn(p, f, 0.9999992847442627f);
#endif
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ float2 ex2_fma_pipe(float2 x) {
#if ASUKA_COL_POLY_SCALAR
  return make_float2(ex2_fma_pipe1(x.x), ex2_fma_pipe1(x.y));
#else
  const float2 magic = make_float2(12582912.f, 12582912.f);
#ifndef ASUKA_COL_POLY_NOCLAMP
  x.x = fmaxf(x.x, -120.f);
  x.y = fmaxf(x.y, -120.f);
#endif
  const float2 t = __fadd2_rn(x, magic);
  const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
#if ASUKA_COL_POLY_DEG == 3
  float2 p = make_float2(0.055171605199575424f, 0.055171605199575424f);
  p = __ffma2_rn(p, f, make_float2(0.2426111102104187f, 0.2426111102104187f));
  p = __ffma2_rn(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
  p = __ffma2_rn(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
#else
  float2 p = make_float2(0.009570094756782055f, 0.009570094756782055f);
  p = __ffma2_rn(p, f, make_float2(0.05591785907745361f, 0.05591785907745361f));
  p = __ffma2_rn(p, f, make_float2(0.240247443318367f, 0.240247443318367f));
  p = __ffma2_rn(p, f, make_float2(0.6931217908859253f, 0.6931217908859253f));
  p = __ffma2_rn(p, f, make_float2(0.9999992847442627f, 0.9999992847442627f));
#endif
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
#endif
}

// Seeded Keyformer noise: one bijective 32-bit mix ("lowbias32") per logit.
//   head_key = hash(seed_lo ^ hash((b*H + h) ^ seed_hi));  word = hash(((q << 16) ^ kv) ^ head_key)
//   u = ((word >> 9) + 0.5) * 2^-23 in (0,1);  exp_rand = -ln(u);  noise g = -ln(exp_rand) ~ Gumbel(0,1)
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ uint32_t seeded_head_key(uint64_t seed, uint32_t bh) {
  return hash_u32(static_cast<uint32_t>(seed) ^ hash_u32(bh ^ static_cast<uint32_t>(seed >> 32)));
}
// log2(exp_rand) of logit (q, kv): exp_rand = -ln(u) = -lg2(u) * ln 2
__device__ __forceinline__ float seeded_lg2_exp_rand(uint32_t q, uint32_t kv, uint32_t head_key) {
  const uint32_t w = hash_u32(((q << 16) ^ kv) ^ head_key);
  const float u = __uint_as_float(0x3f800000u | (w >> 9)) + (-1.0f + 5.9604645e-8f);  // exact
  // -ln(u): the hardware log2 has a fixed ABSOLUTE error, useless for u next to 1 (where the
  // large, row-dominating Gumbel values come from); there use the series in d = 1 - u (exact)
  const float d = 1.0f - u;
  const float series = d * fmaf(d, fmaf(d, 0.33333334f, 0.5f), 1.0f);
  const float er = d < 0.015625f ? series : -0.69314718f * lg2(u);
  return lg2(er);
}

__device__ __forceinline__ void record_timeout(uint32_t* status, uint32_t site) {
  atomicAdd(&status[0], 1u);
  status[1] = site;
}

// kMode: 0 sum, 1 sum + sum of squares, 2 perturbed (noise operand), 3 perturbed (seeded noise),
//        4 CORM: any_i(p_ij >= mask_ij) with a [Sq, Skv] threshold operand (cases/kernels/corm.py:34-37)
template <bool kBF16, int kMode>
__global__ void __launch_bounds__(kThreads, 1)
col_scores_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const ColParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) ColBars bars;
  __shared__ __align__(16) float lse_s[kQStages][kTile];  // minus the row statistic
  __shared__ float part_s[2][2][2][kTile];  // [sum, sum of squares][query half][key tile][key]
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = smem_base;                    // 2 tiles
  const uint32_t sQ = smem_base + 2 * kTileBytes;   // kQStages tiles

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;

  const int bh_count = p.B * p.H;
  const int blk = static_cast<int>(blockIdx.x) / bh_count;
  const int kvb = blk / p.n_qchunks;  // low key blocks are the long ones
  const int qc = p.n_qchunks - 1 - blk % p.n_qchunks;  // (late query ranges see the most keys)
  const int bh = static_cast<int>(blockIdx.x) % bh_count;
  const int b = bh / p.H, h = bh % p.H;
  const int kv0[2] = {kvb * 2 * kTile, kvb * 2 * kTile + kTile};
  const bool active[2] = {kv0[0] < p.Skv, kv0[1] < p.Skv};
  // this CTA's query tiles [i_lo, i_end), and the first of them that can see the first key of
  // each key tile
  const int i_lo = qc * p.q_chunk;
  const int i_end = min(p.nq_tiles, i_lo + p.q_chunk);
  int i_start[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) i_start[t] = max(i_lo, p.causal ? max(0, kv0[t] - p.diag_off) / kTile : 0);
  const int i_begin = i_start[0];
  const int n_active = (active[0] ? 1 : 0) + (active[1] ? 1 : 0);

  // Launched as a programmatic dependent: unless the caller vouches for the kernel ahead (the fused
  // case entry points, whose forward kernel writes only the output and the row statistic), q and k
  // may still be in the making, and everything waits.  Otherwise only the producer waits, before
  // its first read of the row statistic, and the set-up and the K loads run under that kernel's tail.
  if (!p.chained) griddep_wait();
  griddep_launch_dependents();

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&bars.k_full), 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 1 + 8 * n_active);
    }
    for (int t = 0; t < 2; ++t)
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&bars.s_full[t][i]), 1);
        mbar_init(smem_u32(&bars.s_empty[t][i]), 256);
      }
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    // the K tiles are the first thing every role waits for: start them now, under the TMEM
    // allocation and the CTA-wide barrier below (this thread initialised the barrier they signal)
    {
      const uint32_t bar = smem_u32(&bars.k_full);
      mbar_expect_tx(bar, kTileBytes * n_active);
      for (int t = 0; t < 2; ++t) {
        if (active[t]) {
          tma_load_4d(sK + t * kTileBytes, &map_k, bar, 0, h / p.group, kv0[t], b);
          tma_load_4d(sK + t * kTileBytes + kHalfBytes, &map_k, bar, 64, h / p.group, kv0[t], b);
        }
      }
    }
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp)
    const float* lse_row = p.lse2 + (static_cast<size_t>(b) * p.H + h) * p.Sq;
    bool ok = true;
    if (p.chained) griddep_wait();  // the row statistic is the output of the kernel ahead
    for (int i = i_begin; i < i_end; ++i) {
      const int c = i - i_begin;
      const int st = c % kQStages;
      const uint32_t use = static_cast<uint32_t>(c / kQStages);
      if (use > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.q_empty[st]), (use - 1) & 1, abortp));
        if (!ok) { if (lane == 0) record_timeout(p.status, 21); break; }
      }
      // NEGATED row statistics of this query tile (they are only ever subtracted); rows past the
      // end get -inf so that exp2 gives 0
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int qi = i * kTile + r * 32 + lane;
        lse_s[st][r * 32 + lane] = qi < p.Sq ? -__ldg(lse_row + qi) : -INFINITY;
      }
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = smem_u32(&bars.q_full[st]);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sQ + st * kTileBytes, &map_q, bar, 0, h, i * kTile, b);
        tma_load_4d(sQ + st * kTileBytes + kHalfBytes, &map_q, bar, 64, h, i * kTile, b);
      }
    }
    if (!ok && lane == 0) {
      volatile uint32_t none = 0;
      mbar_wait(smem_u32(&bars.k_full), 0, &none);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (warp-uniform descriptors, converged waits); one elected lane
    // issues the tcgen05.mma / commit instructions.
    {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
        const bool good = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, abortp));
        if (!good && lane == 0) record_timeout(p.status, site);
        return good;
      };
      bool ok = wait_all(&bars.k_full, 0, 22);
      for (int i = i_begin; i < i_end && ok; ++i) {
        const int c = i - i_begin;
        const int st = c % kQStages;
        ok = wait_all(&bars.q_full[st], (c / kQStages) & 1, 23);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ + st * kTileBytes, 16, 1024);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!active[t] || i < i_start[t]) continue;
          const int ct = i - i_start[t];
          const int buf = ct & 1;
          if (ct >= 2) {
            ok = wait_all(&bars.s_empty[t][buf], ((ct >> 1) - 1) & 1, 24);
            if (!ok) break;
            tc_fence_after_sync();
          }
          const uint64_t kdesc = umma_smem_desc_sw128(sK + t * kTileBytes, 16, 1024);
          const uint32_t tS = tbase + (t * 2 + buf) * 128;
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
              umma_ss(tS, kdesc + off, qdesc + off, idesc, kk > 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&bars.s_full[t][buf]));
          }
          __syncwarp();
        }
        if (!ok) break;
        if (elect_one()) umma_commit(smem_u32(&bars.q_empty[st]));
        __syncwarp();
      }
    }
  } else if (warp < kUtilWarps) {
  } else {
    // ------------------------------------------------------------------ one thread per (key, query half)
    const int kw = warp - kUtilWarps;
    const int t = kw >> 3;         // key tile
    const int hq = (kw >> 2) & 1;  // which 64 queries of every query tile
    const int wq = warp & 3;       // TMEM lane quarter this warp may touch (every four consecutive key warps cover all four)
    const int key = kv0[t] + wq * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float scale = p.scale_log2;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float acc2[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    const uint32_t head_key = kMode == 3 ? seeded_head_key(p.seed, static_cast<uint32_t>(bh) + p.unit_off) : 0u;
    const float* er_col = nullptr;
    if constexpr (kMode == 2 || kMode == 4) {  // mode 4: the threshold operand, strides 0 for b and h
      er_col = p.exp_rand + static_cast<int64_t>(b) * p.er_sb + static_cast<int64_t>(h) * p.er_sh +
               min(key, p.Skv - 1);
    }
    bool hit = false;

    if (active[t]) {
      for (int i = i_begin; i < i_end; ++i) {
        const int c = i - i_begin;
        const int st = c % kQStages;
        if (i >= i_start[t]) {
          const int ct = i - i_start[t];
          const int buf = ct & 1;
          // S^T of this step is complete; its MMAs were issued after Q and the row statistics of
          // the stage had landed, so this wait covers q_full as well
          ok = __all_sync(0xffffffffu,
                          mbar_wait(smem_u32(&bars.s_full[t][buf]), (ct >> 1) & 1, abortp));
          if (!ok) { if (lane == 0) record_timeout(p.status, 26); break; }
          tc_fence_after_sync();
          const uint32_t tS = tbase + lane_base + (t * 2 + buf) * 128 + hq * 64;
          const int q_base = i * kTile + hq * 64;
          // query q of this tile sees `key` iff key <= q + diag_off
          const int first_visible = p.causal ? key - p.diag_off - q_base : 0;
          const bool tile_has_mask = p.causal && (kv0[t] + kTile - 1 - p.diag_off > q_base);
          const float4* lse4 = reinterpret_cast<const float4*>(lse_s[st]) + hq * 16;
          // two chunks of 32 queries: every exponential of a chunk is in flight at once
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            float s[32];
            tmem_ld32(tS + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(s));
            float noise[(kMode == 2 || kMode == 4) ? 32 : 1];
            if constexpr (kMode == 2 || kMode == 4) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int qi = min(q_base + ch * 32 + e, p.Sq - 1);
                noise[e] = __ldg(er_col + static_cast<int64_t>(qi) * p.er_sq);
              }
              // the operand is read once, straight from HBM: pull the same chunk of the next query
              // tile into L2 now, so that its loads find it there one step later
              if (i + 1 < i_end) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int qi = min(q_base + kTile + ch * 32 + e, p.Sq - 1);
                  asm volatile("prefetch.global.L2 [%0];" ::"l"(er_col + static_cast<int64_t>(qi) * p.er_sq));
                }
              }
            }
            tmem_wait_ld();
            if (ch == 1) {
              // this thread's part of the tile is in registers; when all 256 have said so the MMA
              // warp may overwrite the TMEM buffer
              tc_fence_before_sync();
              mbar_arrive(smem_u32(&bars.s_empty[t][buf]));
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 L = lse4[ch * 8 + g];
              const float lv[4] = {L.x, L.y, L.z, L.w};  // minus the row statistic
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int cc = g * 4 + e;
                float x;
                if constexpr (kMode == 2) {
                  x = fmaf(s[cc], scale, fmaf(lg2(noise[cc]), -p.inv_tau, lv[e]));
                } else if constexpr (kMode == 3) {
                  const float l2 = seeded_lg2_exp_rand(static_cast<uint32_t>(q_base + ch * 32 + cc),
                                                       static_cast<uint32_t>(key), head_key);
                  x = fmaf(s[cc], scale, fmaf(l2, -p.inv_tau, lv[e]));
                } else {
                  x = 0.f;  // (modes 0, 1, 4 take the packed path below)
                }
                if constexpr (kMode == 2 || kMode == 3) s[cc] = ex2(x);
              }
              if constexpr (kMode != 2 && kMode != 3) {
                // two logits per FMA instruction (packed f32x2 of sm_100)
                const float2 sc2 = make_float2(scale, scale);
                const float2 x01 = __ffma2_rn(make_float2(s[g * 4 + 0], s[g * 4 + 1]), sc2, make_float2(lv[0], lv[1]));
                const float2 x23 = __ffma2_rn(make_float2(s[g * 4 + 2], s[g * 4 + 3]), sc2, make_float2(lv[2], lv[3]));
                // pairs alternate between the MUFU and the FMA pipe in the configured proportion
                constexpr int kQ = ASUKA_COL_POLY_QUARTERS;
                const bool poly01b = kQ == 3 && (g & 1) != 0;
                const bool poly23 = kQ >= 2 || (kQ == 1 && (g & 1) != 0);
                if (poly01b) {
                  const float2 e01 = ex2_fma_pipe(x01);
                  s[g * 4 + 0] = e01.x;
                  s[g * 4 + 1] = e01.y;
                } else {
                  s[g * 4 + 0] = ex2(x01.x);
                  s[g * 4 + 1] = ex2(x01.y);
                }
                if (poly23) {
                  const float2 e23 = ex2_fma_pipe(x23);
                  s[g * 4 + 2] = e23.x;
                  s[g * 4 + 3] = e23.y;
                } else {
                  s[g * 4 + 2] = ex2(x23.x);
                  s[g * 4 + 3] = ex2(x23.y);
                }
              }
            }
            if (tile_has_mask) {
#pragma unroll
              for (int cc = 0; cc < 32; ++cc) s[cc] = (ch * 32 + cc < first_visible) ? 0.f : s[cc];
            }
            if constexpr (kMode == 4) {
#pragma unroll
              for (int cc = 0; cc < 32; ++cc) hit = hit || (s[cc] >= noise[cc] && q_base + ch * 32 + cc < p.Sq);
            } else {
              float2 a01 = make_float2(acc[0], acc[1]), a23 = make_float2(acc[2], acc[3]);
              float2 q01 = make_float2(acc2[0], acc2[1]), q23 = make_float2(acc2[2], acc2[3]);
#pragma unroll
              for (int cc = 0; cc < 32; cc += 4) {
                const float2 p01 = make_float2(s[cc], s[cc + 1]), p23 = make_float2(s[cc + 2], s[cc + 3]);
                a01 = __fadd2_rn(a01, p01);
                a23 = __fadd2_rn(a23, p23);
                if constexpr (kMode == 1) {
                  q01 = __ffma2_rn(p01, p01, q01);
                  q23 = __ffma2_rn(p23, p23, q23);
                }
              }
              acc[0] = a01.x; acc[1] = a01.y; acc[2] = a23.x; acc[3] = a23.y;
              acc2[0] = q01.x; acc2[1] = q01.y; acc2[2] = q23.x; acc2[3] = q23.y;
            }
          }
        } else {
          // a step this key tile skips (its keys are invisible to the whole query tile): the stage
          // may only be released once it has been filled
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.q_full[st]), (c / kQStages) & 1, abortp));
          if (!ok) { if (lane == 0) record_timeout(p.status, 25); break; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.q_empty[st]));
      }
    }
    // Both query halves leave their parts in shared memory; after the CTA-wide barrier below the
    // first half's thread adds the two in a fixed order and stores.
    part_s[0][hq][t][wq * 32 + lane] = kMode == 4 ? (hit ? 1.f : 0.f) : (acc[0] + acc[1]) + (acc[2] + acc[3]);
    part_s[1][hq][t][wq * 32 + lane] = (acc2[0] + acc2[1]) + (acc2[2] + acc2[3]);
    if (!ok) *abortp = 1u;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 512);
  }
  if (warp >= kUtilWarps && ((warp - kUtilWarps) >> 2 & 1) == 0 && !*abortp) {
    const int t = (warp - kUtilWarps) >> 3;
    const int k_in_tile = (warp & 3) * 32 + lane;
    const int key = kv0[t] + k_in_tile;
    if (key < p.Skv) {  // (implies that this key tile is active)
      const size_t o = (static_cast<size_t>(b) * p.H + h) * p.Skv + key;
      const float v = part_s[0][0][t][k_in_tile] + part_s[0][1][t][k_in_tile];
      // with a query-range split the sums of this range go to its slab of the workspace (a range
      // that sees none of the keys leaves zeros there)
      const size_t slab = static_cast<size_t>(qc) * bh_count * p.Skv;
      if constexpr (kMode == 4) {
        reinterpret_cast<uint8_t*>(p.score)[o] = v != 0.f ? 1 : 0;
      } else {
        (p.n_qchunks > 1 ? p.part + slab : p.score)[o] = v;
      }
      if constexpr (kMode == 1)
        (p.n_qchunks > 1 ? p.part_sq + slab : p.score_sq)[o] = part_s[1][0][t][k_in_tile] + part_s[1][1][t][k_in_tile];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Keyformer column pass with the noise operand staged by TMA.
// The operand is read exactly once and is nine tenths of this pass's traffic; a thread that owns a
// key (the transposed layout the MMA gives) would read its column of it with scalar loads, one
// round trip to L2 or DRAM per 32 logits.  Here a CTA owns ONE key tile, which leaves shared
// memory for a ring of four noise pieces [64 queries x 128 keys] f32 (four 128-byte-swizzled boxes
// of 32 keys each, as in the row pass); three pieces are in flight while one is consumed (with two
// in flight the pass ran at 4.7 TB/s: 64 KB per SM do not cover the latency of DRAM under load).  The sixteen
// key warps are (TMEM lane quarter) x (16 of a piece's 64 queries).  A CTA takes two key tiles in
// turn (see the comment on segments in the kernel).
// ---------------------------------------------------------------------------------------------
constexpr int kNzQStages = 2;
constexpr int kNzStages = 4;
constexpr int kNzRows = 64;                                  // queries per noise piece
constexpr uint32_t kNzPieceBytes = kNzRows * kTile * 4;      // 32 KB
constexpr uint32_t kNzBoxBytes = kNzPieceBytes / 4;          // one box: 32 keys x 64 queries
constexpr uint32_t kNzSmemBytes = (1 + kNzQStages) * kTileBytes + kNzStages * kNzPieceBytes + 1024;

struct NzBars {
  uint64_t k_full;
  uint64_t q_full[kNzQStages], q_empty[kNzQStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t n_full[kNzStages], n_empty[kNzStages];
};

template <bool kBF16>
__global__ void __launch_bounds__(kThreads, 1)
kf_col_tma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_n, const ColParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) NzBars bars;
  __shared__ __align__(16) float lse_s[kNzQStages][kTile];  // minus the row statistic
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base;
  const uint32_t sQ = smem_base + kTileBytes;
  const uint32_t sN = sQ + kNzQStages * kTileBytes;
  // [segment][which 16 queries][key] partial sums, written after a warp's last step: they take the
  // place of the first Q stage, which nothing reads any more by then (every MMA has retired
  // before the step that waits for it is over, and no copy into the stage is outstanding)
  float (*part_s)[4][kTile] = reinterpret_cast<float (*)[4][kTile]>(smem_raw + (sQ - smem_u32(smem_raw)));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;

  // Unit-major grid: the key tiles of one (batch, head) run at about the same time, so that Q,
  // which every one of them reads, comes from DRAM once (the noise streaming through L2 would
  // have pushed it out by the time a later wave asked for it again).
  // A CTA works through TWO key tiles, one after the other ("segments"): tile i and tile
  // n - 1 - i, which under a causal mask together always make n + 1 steps, so all CTAs are equally
  // long and there are half as many set-ups and drains.  The Q, noise and TMEM rings run on
  // across the change of segment; only K is reloaded, while the key warps still work on the
  // first segment's last step.
  const int bh_count = p.B * p.H;
  const int n_kt = (p.Skv + kTile - 1) / kTile;
  const int per_unit = static_cast<int>(gridDim.x) / bh_count;  // pairs of key tiles x query ranges
  const int blk = static_cast<int>(blockIdx.x) % per_unit;
  const int pair = blk / p.n_qchunks;
  const int qc = p.n_qchunks - 1 - blk % p.n_qchunks;  // (late query ranges see the most keys)
  const int bh = static_cast<int>(blockIdx.x) / per_unit;
  const int b = bh / p.H, h = bh % p.H;
  const int kts[2] = {pair, n_kt - 1 - pair};
  const int n_seg = kts[1] > kts[0] ? 2 : 1;  // (an odd count leaves the middle tile alone)
  const int i_lo = qc * p.q_chunk;
  const int i_end = min(p.nq_tiles, i_lo + p.q_chunk);
  // first key, first query tile of this CTA's range that can see it, and number of steps of segment s
  auto segment = [&](int sgm, int& kv0, int& i_begin, int& n_steps) {
    kv0 = kts[sgm] * kTile;
    i_begin = max(i_lo, p.causal ? max(0, kv0 - p.diag_off) / kTile : 0);
    n_steps = max(0, i_end - i_begin);
  };

  if (!p.chained) griddep_wait();
  griddep_launch_dependents();

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&bars.k_full), 1);
    for (int i = 0; i < kNzQStages; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 1 + 16);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.s_empty[i]), 512);
    }
    for (int i = 0; i < kNzStages; ++i) {
      mbar_init(smem_u32(&bars.n_full[i]), 1);
      mbar_init(smem_u32(&bars.n_empty[i]), 16);
    }
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_n);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;

  // Steps and noise pieces are counted through both segments: ring stages and barrier parities
  // follow from the running counts.
  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp)
    // Order of issue within a segment: K; Q of its first step; then per step its two noise
    // pieces, then Q of the next step.  A noise piece waits for the piece four before it to have
    // been consumed, Q of step c + 1 for step c - 1 to be over: while the key warps work on step
    // c the pieces of step c + 1 are in flight, and Q of step c + 1 arrives as well.
    const float* lse_row = p.lse2 + (static_cast<size_t>(b) * p.H + h) * p.Sq;
    bool ok = true;
    if (p.chained) griddep_wait();  // the row statistic is the output of the kernel ahead
    auto load_q = [&](uint32_t cg, int i) -> bool {  // cg: running step count, i: query tile
      const int st = cg % kNzQStages;
      const uint32_t use = cg / kNzQStages;
      if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.q_empty[st]), (use - 1) & 1, abortp))) {
        if (lane == 0) record_timeout(p.status, 61);
        return false;
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int qi = i * kTile + r * 32 + lane;
        lse_s[st][r * 32 + lane] = qi < p.Sq ? -__ldg(lse_row + qi) : -INFINITY;
      }
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = smem_u32(&bars.q_full[st]);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sQ + st * kTileBytes, &map_q, bar, 0, h, i * kTile, b);
        tma_load_4d(sQ + st * kTileBytes + kHalfBytes, &map_q, bar, 64, h, i * kTile, b);
      }
      return true;
    };
    uint32_t issued = 0;   // noise pieces issued
    uint32_t cg0 = 0;      // steps of the segments before this one
    uint32_t k_loads = 0;
    const uint64_t stream_once = l2_policy_evict_first();
    for (int sgm = 0; sgm < n_seg && ok; ++sgm) {
      int kv0, i_begin, n_steps;
      segment(sgm, kv0, i_begin, n_steps);
      if (n_steps == 0) continue;
      if (cg0 > 0) {
        // the K buffer is free once the last MMA that read it has retired
        const uint32_t last = cg0 - 1;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.s_full[last & 1]), (last >> 1) & 1, abortp))) {
          if (lane == 0) record_timeout(p.status, 68);
          ok = false;
          break;
        }
      }
      if (lane == 0) {
        const uint32_t bar = smem_u32(&bars.k_full);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sK, &map_k, bar, 0, h / p.group, kv0, b);
        tma_load_4d(sK + kHalfBytes, &map_k, bar, 64, h / p.group, kv0, b);
      }
      ++k_loads;
      __syncwarp();
      ok = load_q(cg0, i_begin);
      for (int c = 0; c < n_steps && ok; ++c) {
        const int i = i_begin + c;
        for (int pc = 0; pc < 2 && ok; ++pc, ++issued) {
          const int ns = issued % kNzStages;
          const uint32_t use = issued / kNzStages;
          if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.n_empty[ns]), (use - 1) & 1, abortp))) {
            if (lane == 0) record_timeout(p.status, 62);
            ok = false;
            break;
          }
          if (lane == 0) {
            const uint32_t bar = smem_u32(&bars.n_full[ns]);
            // boxes whose first key no query of the piece can see are not fetched (their threads
            // mask every value of the piece); the operand is read once: first to leave L2
            const int q_last = i * kTile + pc * kNzRows + kNzRows - 1;
            int n_vis = 4;
            if (p.causal) {
              const int d = q_last + p.diag_off - kv0;  // last visible key of the piece, relative to the tile
              n_vis = d < 0 ? 0 : min(4, d / 32 + 1);
            }
            mbar_expect_tx(bar, n_vis * kNzBoxBytes);
            for (int w = 0; w < n_vis; ++w)
              tma_load_4d_hint(sN + ns * kNzPieceBytes + w * kNzBoxBytes, &map_n, bar, kv0 + w * 32,
                               i * kTile + pc * kNzRows, h, b, stream_once);
          }
          __syncwarp();
        }
        if (ok && c + 1 < n_steps) ok = load_q(cg0 + c + 1, i + 1);
      }
      cg0 += static_cast<uint32_t>(n_steps);
    }
    if (!ok && lane == 0) {
      // give copies already in flight a bounded chance to land before the CTA retires
      volatile uint32_t none = 0;
      if (k_loads > 0) mbar_wait(smem_u32(&bars.k_full), (k_loads - 1) & 1, &none);
      for (uint32_t x = issued > kNzStages ? issued - kNzStages : 0; x < issued; ++x)
        mbar_wait(smem_u32(&bars.n_full[x % kNzStages]), (x / kNzStages) & 1, &none);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
    constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
    auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
      const bool good = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, abortp));
      if (!good && lane == 0) record_timeout(p.status, site);
      return good;
    };
    bool ok = true;
    uint32_t cg0 = 0, k_loads = 0;
    const uint64_t kdesc = umma_smem_desc_sw128(sK, 16, 1024);
    for (int sgm = 0; sgm < n_seg && ok; ++sgm) {
      int kv0, i_begin, n_steps;
      segment(sgm, kv0, i_begin, n_steps);
      if (n_steps == 0) continue;
      ok = wait_all(&bars.k_full, k_loads & 1, 63);
      ++k_loads;
      for (int c = 0; c < n_steps && ok; ++c) {
        const uint32_t cg = cg0 + c;
        const int st = cg % kNzQStages, buf = cg & 1;
        ok = wait_all(&bars.q_full[st], (cg / kNzQStages) & 1, 64);
        if (!ok) break;
        if (cg >= 2) {
          ok = wait_all(&bars.s_empty[buf], ((cg >> 1) - 1) & 1, 65);
          if (!ok) break;
        }
        tc_fence_after_sync();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ + st * kTileBytes, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
            umma_ss(tbase + buf * 128, kdesc + off, qdesc + off, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars.s_full[buf]));
          umma_commit(smem_u32(&bars.q_empty[st]));
        }
        __syncwarp();
      }
      cg0 += static_cast<uint32_t>(n_steps);
    }
  } else {
    // ------------------------------------------------------------------ one thread per (key, 16 of every 64 queries)
    const int kw = warp - kUtilWarps;
    const int sub = kw >> 2;   // which 16 queries of every piece
    const int wq = warp & 3;   // TMEM lane quarter this warp may touch (four consecutive warps cover all four)
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float scale = p.scale_log2;
    const float neg_inv_tau = -p.inv_tau;
    bool ok = true;
    uint32_t nc = 0;   // noise pieces consumed
    uint32_t cg0 = 0;  // steps of the segments before this one
    float seg_sum[2] = {0.f, 0.f};
    for (int sgm = 0; sgm < n_seg; ++sgm) {
      int kv0, i_begin, n_steps;
      segment(sgm, kv0, i_begin, n_steps);
      const int key = kv0 + wq * 32 + lane;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < n_steps && ok; ++c) {
        const int i = i_begin + c;
        const uint32_t cg = cg0 + c;
        const int st = cg % kNzQStages, buf = cg & 1;
        // S^T of this step is complete; its MMAs were issued after Q and the row statistics of the
        // stage had landed, so this wait covers q_full as well
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.s_full[buf]), (cg >> 1) & 1, abortp));
        if (!ok) { if (lane == 0) record_timeout(p.status, 66); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int pc = 0; pc < 2; ++pc, ++nc) {
          const int ns = nc % kNzStages;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.n_full[ns]), (nc / kNzStages) & 1, abortp));
          if (!ok) { if (lane == 0) record_timeout(p.status, 67); break; }
          const int col0 = pc * kNzRows + sub * 16;  // first of this thread's 16 queries within the tile
          uint32_t u[16];
          tmem_ld16(tbase + lane_base + buf * 128 + col0, u);
          // the thread's key is column `lane` of box wq; its queries are rows sub*16 .. +15
          const uint8_t* box = smem_gen + (sN - smem_base) + ns * kNzPieceBytes + wq * kNzBoxBytes;
          float nz[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int r = sub * 16 + e;
            nz[e] = *reinterpret_cast<const float*>(box + sw128_offset(r, lane >> 2) + (lane & 3) * 4);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.n_empty[ns]));
          tmem_wait_ld();
          if (pc == 1) {
            // this thread's part of the tile is in registers; when all 512 have said so the MMA
            // warp may overwrite the TMEM buffer
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars.s_empty[buf]));
          }
          const int q_base = i * kTile + col0;
          // query q sees `key` iff key <= q + diag_off
          const int first_visible = p.causal ? key - p.diag_off - q_base : 0;
          const float4* lse4 = reinterpret_cast<const float4*>(lse_s[st]) + (col0 >> 2);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const float4 L = lse4[g];
            const float lv[4] = {L.x, L.y, L.z, L.w};  // minus the row statistic (-inf past the last query)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int cc = g * 4 + e;
              // (rows and keys past the tensor's end are zero-filled by the copy: keep lg2 finite,
              // the row statistic of -inf or the bounds check at the end removes them)
              const float l2 = lg2(fmaxf(nz[cc], 1e-30f));
              const float x = fmaf(__uint_as_float(u[cc]), scale, fmaf(l2, neg_inv_tau, lv[e]));
              const float pr = cc < first_visible ? 0.f : ex2(x);
              acc[e] += pr;
            }
          }
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.q_empty[st]));
      }
      cg0 += static_cast<uint32_t>(n_steps);
      seg_sum[sgm] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
    // (only now: the partial sums lie over a Q stage, which the second segment still uses)
    part_s[0][sub][wq * 32 + lane] = seg_sum[0];
    part_s[1][sub][wq * 32 + lane] = seg_sum[1];
    if (!ok) *abortp = 1u;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 256);
  }
  if (warp >= kUtilWarps && ((warp - kUtilWarps) >> 2) == 0 && !*abortp) {
    const int k_in_tile = (warp & 3) * 32 + lane;
    for (int sgm = 0; sgm < n_seg; ++sgm) {
      const int key = kts[sgm] * kTile + k_in_tile;
      if (key < p.Skv) {
        const size_t o = (static_cast<size_t>(b) * p.H + h) * p.Skv + key;
        const float v = (part_s[sgm][0][k_in_tile] + part_s[sgm][1][k_in_tile]) +
                        (part_s[sgm][2][k_in_tile] + part_s[sgm][3][k_in_tile]);
        const size_t slab = static_cast<size_t>(qc) * bh_count * p.Skv;
        (p.n_qchunks > 1 ? p.part + slab : p.score)[o] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Keyformer row pass: lse2'[row] = log2 sum_j exp2(((s_ij*scale + g_ij)/tau) * log2e)
// One CTA per 128 query rows; one thread per row; K tiles stream through a ring.
// kNoiseTma: the [128 x 128] f32 noise tile of every step is staged in shared memory by TMA
// (four 128-byte-swizzled boxes of 32 keys) -- the kernel is bound by that 2 GB read, and a
// thread walking its own row in global memory wastes most of every sector.  The boxes of two steps
// form a ring of eight with a barrier pair each: a box goes back to the producer as soon as the
// four warps that read it have it in registers, so the first boxes of the step after next are
// under way while the second half of the current step is computed (what is in flight per SM is
// what bounds a pass that reads everything once).  The plain variant (direct loads) serves noise
// tensors whose strides TMA cannot describe.
// ---------------------------------------------------------------------------------------------
constexpr int kRsThreads = 320;  // warp 0 producer, warp 1 MMA, warps 2-9 rows (two per 32 rows: columns 0..63 / 64..127)
constexpr uint32_t kNoiseTileBytes = 128 * 128 * 4;
constexpr uint32_t kNoiseBoxBytes = kNoiseTileBytes / 4;
template <int kNoise> struct RsCfg {  // kNoise 1: two K stages, then eight noise boxes
  static constexpr bool kNoiseTma = kNoise == 1;
  static constexpr int kStages = kNoise == 0 ? 4 : 2;  // seeded: small enough for two CTAs per SM
  static constexpr uint32_t kStageBytes = kTileBytes + (kNoiseTma ? kNoiseTileBytes : 0);
  static constexpr uint32_t kSmem = kTileBytes + kStages * kStageBytes + 1024;
};

struct RsBars {
  uint64_t q_full;
  uint64_t k_full[4], k_empty[4];
  uint64_t s_full[2], s_empty[2];
  uint64_t n_full[8], n_empty[8];  // staged noise: one pair per box of the ring
};

// kNoise: 0 noise operand read directly, 1 noise operand staged by TMA, 2 seeded noise
template <bool kBF16, int kNoise>
__global__ void __launch_bounds__(kRsThreads, kNoise == 2 ? 2 : 1)
kf_rowstat_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_n, const ColParams p, float* lse_out) {
  constexpr bool kNoiseTma = kNoise == 1;
  using Cfg = RsCfg<kNoise>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) RsBars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sStage = smem_base + kTileBytes;             // the K stages
  const uint32_t sNoise = sStage + kStages * kTileBytes;      // (TMA variant) eight boxes [128 rows x 32 keys] f32

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;
  const int bh_count = p.B * p.H;
  // Unit-major grid: the query tiles of one (batch, head) run at about the same time, latest
  // (longest) first, so that K, which every one of them reads, comes from DRAM once -- with two
  // gigabytes of noise streaming through L2 it does not survive from one wave to a later one
  // (measured before the change: 1.65 GB read where 1.27 GB were needed).
  // The seeded variant reads no operand and is bound by its generator: it keeps the order
  // longest tile first over all units, which balances the SMs better.
  constexpr bool kUnitMajor = kNoise != 2;
  const int bh = kUnitMajor ? static_cast<int>(blockIdx.x) / p.nq_tiles : static_cast<int>(blockIdx.x) % bh_count;
  const int qt = p.nq_tiles - 1 - (kUnitMajor ? static_cast<int>(blockIdx.x) % p.nq_tiles
                                              : static_cast<int>(blockIdx.x) / bh_count);
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qt * kTile;
  int last = p.Skv - 1;
  if (p.causal) last = min(last, min(q0 + kTile - 1, p.Sq - 1) + p.diag_off);
  const int n_kv = last / kTile + 1;

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&bars.q_full), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bars.k_full[i]), 1);
      mbar_init(smem_u32(&bars.k_empty[i]), 1);  // the MMA commit
    }
    if constexpr (kNoiseTma) {
      for (int i = 0; i < 8; ++i) {
        mbar_init(smem_u32(&bars.n_full[i]), 1);
        mbar_init(smem_u32(&bars.n_empty[i]), 4);  // the four warps that read the box
      }
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.s_empty[i]), 256);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      {
        const uint32_t bar = smem_u32(&bars.q_full);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sQ, &map_q, bar, 0, h, q0, b);
        tma_load_4d(sQ + kHalfBytes, &map_q, bar, 64, h, q0, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % kStages;
        const uint32_t use = static_cast<uint32_t>(j / kStages);
        if (use > 0 && !mbar_wait(smem_u32(&bars.k_empty[st]), (use - 1) & 1, abortp)) {
          record_timeout(p.status, 31);
          break;
        }
        const uint32_t bar = smem_u32(&bars.k_full[st]);
        const uint32_t base = sStage + st * kTileBytes;
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(base, &map_k, bar, 0, h / p.group, j * kTile, b);
        tma_load_4d(base + kHalfBytes, &map_k, bar, 64, h / p.group, j * kTile, b);
        if constexpr (kNoiseTma) {
          // the first box of either column half first; step j uses ring slots (j & 1) * 4 ..
          bool good = true;
#pragma unroll
          for (int x = 0; x < 4 && good; ++x) {
            const int c4 = (x & 1) * 2 + (x >> 1);  // 0, 2, 1, 3
            const int slot = (j & 1) * 4 + c4;
            if (j >= 2 && !mbar_wait(smem_u32(&bars.n_empty[slot]), ((j >> 1) - 1) & 1, abortp)) {
              record_timeout(p.status, 36);
              good = false;
              break;
            }
            const uint32_t nbar = smem_u32(&bars.n_full[slot]);
            mbar_expect_tx(nbar, kNoiseBoxBytes);
            tma_load_4d_hint(sNoise + slot * kNoiseBoxBytes, &map_n, nbar, j * kTile + c4 * 32, q0, h, b,
                             l2_policy_evict_first());  // (read once: first to leave L2)
          }
          if (!good) break;
        }
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
        const bool good = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, abortp));
        if (!good && lane == 0) record_timeout(p.status, site);
        return good;
      };
      bool ok = wait_all(&bars.q_full, 0, 32);
      const uint64_t qdesc = umma_smem_desc_sw128(sQ, 16, 1024);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % kStages, buf = j & 1;
        ok = wait_all(&bars.k_full[st], (j / kStages) & 1, 33);
        if (!ok) break;
        if (j >= 2) {
          ok = wait_all(&bars.s_empty[buf], ((j >> 1) - 1) & 1, 34);
          if (!ok) break;
        }
        tc_fence_after_sync();
        const uint64_t kdesc = umma_smem_desc_sw128(sStage + st * kTileBytes, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
            umma_ss(tbase + buf * 128, qdesc + off, kdesc + off, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars.s_full[buf]));
          umma_commit(smem_u32(&bars.k_empty[st]));
        }
        __syncwarp();
      }
    }
  } else {
    // Two warps per 32 rows, each with half of every tile's columns and its own running (maximum,
    // sum): a row's statistic is a plain merge of the two at the end, so nothing is exchanged per
    // step, and the scheduler gets twice the warps to hide the noise generator's ALU latency.
    const int wq = warp & 3;           // TMEM lane quarter (warps 2..9 -> 2,3,0,1,2,3,0,1)
    const int half = (warp - 2) >> 2;  // columns 0..63 or 64..127 of every tile
    const int r_in_tile = wq * 32 + lane;
    const int row = q0 + r_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    int lim = p.Skv - 1;
    if (p.causal) lim = min(lim, row + p.diag_off);
    const float scale = p.scale_log2;
    const float* er_row = kNoise == 2 ? nullptr
                                      : p.exp_rand + static_cast<int64_t>(b) * p.er_sb +
                                            static_cast<int64_t>(h) * p.er_sh +
                                            static_cast<int64_t>(min(row, p.Sq - 1)) * p.er_sq;
    const uint32_t head_key = kNoise == 2 ? seeded_head_key(p.seed, static_cast<uint32_t>(bh) + p.unit_off) : 0u;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int buf = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.s_full[buf]), (j >> 1) & 1, abortp));
      if (!ok) { if (lane == 0) record_timeout(p.status, 35); break; }
      tc_fence_after_sync();
      const int thr = lim - j * kTile;  // columns > thr are masked
#pragma unroll
      for (int c4 = half * 2; c4 < half * 2 + 2; ++c4) {
        uint32_t u[32];
        tmem_ld32(tbase + lane_base + buf * 128 + c4 * 32, u);
        float er[32];
        if constexpr (kNoiseTma) {
          const int slot = (j & 1) * 4 + c4;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.n_full[slot]), (j >> 1) & 1, abortp));
          if (!ok) { if (lane == 0) record_timeout(p.status, 37); break; }
          // this row's 32 noise values of box c4: eight swizzled 16-byte chunks
          const uint8_t* box = smem_gen + (sNoise - smem_base) + slot * kNoiseBoxBytes;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const float4 v = *reinterpret_cast<const float4*>(box + sw128_offset(r_in_tile, ch));
            er[ch * 4 + 0] = v.x; er[ch * 4 + 1] = v.y; er[ch * 4 + 2] = v.z; er[ch * 4 + 3] = v.w;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.n_empty[slot]));  // in registers: the box may be refilled
        } else if constexpr (kNoise == 0) {
#pragma unroll
          for (int e = 0; e < 32; ++e) er[e] = __ldg(er_row + min(j * kTile + c4 * 32 + e, p.Skv - 1));
        }
        tmem_wait_ld();
        float x[32];
        float mt4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int cc = c4 * 32 + e;
          float l2;
          if constexpr (kNoise == 2) {
            l2 = seeded_lg2_exp_rand(static_cast<uint32_t>(row), static_cast<uint32_t>(j * kTile + cc), head_key);
          } else {
            l2 = lg2(er[e]);
          }
          const float v = fmaf(__uint_as_float(u[e]), scale, -l2 * p.inv_tau);
          x[e] = (cc > thr) ? -INFINITY : v;
          mt4[e & 3] = fmaxf(mt4[e & 3], x[e]);
        }
        const float m_new = fmaxf(m, fmaxf(fmaxf(mt4[0], mt4[1]), fmaxf(mt4[2], mt4[3])));
        if (m_new > -INFINITY) {
          float l4[4] = {l * ex2(m - m_new), 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 32; ++e) l4[e & 3] += ex2(x[e] - m_new);
          l = (l4[0] + l4[1]) + (l4[2] + l4[3]);
          m = m_new;
        }
      }
      if (!ok) break;
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars.s_empty[buf]));
    }
    // hand-over through the Q tile's shared memory: every MMA that read it has retired (this thread
    // has seen the last S tile), and the variant with the staged noise has no other room left
    float* part = reinterpret_cast<float*>(smem_gen);  // [m, l][half][row]
    part[(0 * 2 + half) * kTile + r_in_tile] = m;
    part[(1 * 2 + half) * kTile + r_in_tile] = l;
    if (!ok) *abortp = 1u;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 256);
  }
  if (warp >= 2 && warp < 6 && !*abortp) {
    // merge the two halves of every row (in column order)
    const int r_in_tile = (warp & 3) * 32 + lane;
    const int row = q0 + r_in_tile;
    const float* part = reinterpret_cast<const float*>(smem_gen);
    const float m0 = part[0 * kTile + r_in_tile], m1 = part[1 * kTile + r_in_tile];
    const float m = fmaxf(m0, m1);
    if (row < p.Sq) {
      // (a half with no visible column has sum 0 and maximum -inf: give it weight 0, not NaN)
      const float l = part[2 * kTile + r_in_tile] * (m0 > -INFINITY ? ex2(m0 - m) : 0.f) +
                      part[3 * kTile + r_in_tile] * (m1 > -INFINITY ? ex2(m1 - m) : 0.f);
      lse_out[(static_cast<size_t>(b) * p.H + h) * p.Sq + row] = m + log2f(l);
    }
  }
}

// Adds the partial sums of a query-range split in range order: out[i] = sum_c part[c][i].
__global__ void __launch_bounds__(256) sum_chunks_kernel(const float* __restrict__ part, const float* __restrict__ part_sq,
                                                         float* __restrict__ out, float* __restrict__ out_sq,
                                                         int n_chunks, size_t n) {
  griddep_wait();  // the partial sums are the output of the kernel ahead
  griddep_launch_dependents();
  const size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n) return;
  float a = 0.f, q = 0.f;
  for (int c = 0; c < n_chunks; ++c) {
    a += part[c * n + i];
    if (part_sq != nullptr) q += part_sq[c * n + i];
  }
  out[i] = a;
  if (part_sq != nullptr) out_sq[i] = q;
}

ColParams make_params(const ScoreArgs& a, const AttnShape& s) {
  ColParams p;
  p.B = s.B;
  p.H = s.H;
  p.Sq = s.Sq;
  p.Skv = s.Skv;
  p.causal = s.causal;
  p.diag_off = s.Skv - s.Sq;
  p.nq_tiles = (s.Sq + kTile - 1) / kTile;
  p.group = s.group;
  const float log2e = 1.4426950408889634f;
  p.inv_tau = 1.0f;
  p.scale_log2 = s.softmax_scale * log2e;
  if (a.mode == ASUKA_SCORE_PERTURBED) {
    p.inv_tau = 1.0f / a.tau;
    p.scale_log2 = s.softmax_scale * log2e / a.tau;
  }
  p.lse2 = a.lse2;
  p.score = a.score;
  p.score_sq = a.score_sq;
  p.exp_rand = a.exp_rand;
  p.er_sb = a.er_stride_b;
  p.er_sh = a.er_stride_h;
  p.er_sq = a.er_stride_q;
  p.seed = a.seed;
  p.unit_off = a.unit_offset;
  p.status = device_status_words();
  p.chained = a.chained;
  p.q_chunk = p.nq_tiles;
  p.n_qchunks = 1;
  p.part = nullptr;
  p.part_sq = nullptr;
  return p;
}

}  // namespace

// Query ranges the column pass is worth cutting into on `num_sms` SMs (1: no split); every range
// needs a [B*H, Skv] f32 slab of workspace per score tensor.
int col_scores_chunks(const AttnShape& s, int mode, int num_sms, size_t ws_bytes) {
  if (mode == ASUKA_SCORE_CORM) return 1;
  const long long n_ctas = static_cast<long long>((s.Skv + 2 * kTile - 1) / (2 * kTile)) * s.B * s.H;
  const int nq_tiles = (s.Sq + kTile - 1) / kTile;
  int chunks = 1;
#ifdef ASUKA_TUNE_ENV
  if (const char* e = getenv("ASUKA_COL_CHUNKS")) {
    chunks = atoi(e);
    while (chunks > 1 && col_scores_split_bytes(s, mode, chunks) > ws_bytes) chunks /= 2;
    return chunks;
  }
#endif
  // measured at head counts of 4 to 32 and S = 1024 to 4096: worth it only for long query ranges
  // and clearly fewer key blocks than the SMs can take in one wave and a bit
  if (5 * n_ctas < 6LL * num_sms && nq_tiles >= 32) chunks = 2 * n_ctas <= num_sms ? 4 : 2;
  while (chunks > 1 && col_scores_split_bytes(s, mode, chunks) > ws_bytes) chunks /= 2;
  return chunks;
}

size_t col_scores_split_bytes(const AttnShape& s, int mode, int chunks) {
  if (chunks <= 1) return 0;
  const size_t slab = static_cast<size_t>(s.B) * s.H * s.Skv * sizeof(float);
  return slab * chunks * (mode == ASUKA_SCORE_SUM_SQ ? 2 : 1);
}

cudaError_t launch_col_scores(const CUtensorMap& mq, const CUtensorMap& mk, const ScoreArgs& a,
                              const AttnShape& s, void* split_ws, int chunks, cudaStream_t stream,
                              PendingChunkSum* pending) {
  ColParams p = make_params(a, s);
  if (pending != nullptr) pending->n_chunks = 0;
  if (chunks > 1 && split_ws != nullptr && a.mode != ASUKA_SCORE_CORM) {
    p.q_chunk = (p.nq_tiles + chunks - 1) / chunks;
    p.n_qchunks = (p.nq_tiles + p.q_chunk - 1) / p.q_chunk;
    p.part = static_cast<float*>(split_ws);
    p.part_sq = p.part + static_cast<size_t>(p.n_qchunks) * s.B * s.H * s.Skv;
  }
  cudaError_t e;
#ifndef ASUKA_COL_NO_NOISE_TMA
  // Keyformer with a noise operand that TMA can describe (16-byte aligned base, strides that are
  // multiples of 16 bytes): the variant that stages the operand in shared memory
  if (a.mode == ASUKA_SCORE_PERTURBED && a.exp_rand != nullptr &&
      (reinterpret_cast<uintptr_t>(a.exp_rand) & 15u) == 0 && a.er_stride_q % 4 == 0 && a.er_stride_h % 4 == 0 &&
      a.er_stride_b % 4 == 0 && a.er_stride_q > 0 && a.er_stride_h > 0 && a.er_stride_b > 0) {
    CUtensorMap mn;
    const uint64_t dims[4] = {static_cast<uint64_t>(s.Skv), static_cast<uint64_t>(s.Sq),
                              static_cast<uint64_t>(s.H), static_cast<uint64_t>(s.B)};
    const uint64_t strides[3] = {static_cast<uint64_t>(a.er_stride_q) * 4, static_cast<uint64_t>(a.er_stride_h) * 4,
                                 static_cast<uint64_t>(a.er_stride_b) * 4};
    const uint32_t box[4] = {32, kNzRows, 1, 1};
    if (tma_host::make_f32_map_sw128(&mn, a.exp_rand, dims, strides, box) != 0) return cudaErrorInvalidValue;
    auto nk = s.bf16 ? kf_col_tma_kernel<true> : kf_col_tma_kernel<false>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(nk), kNzSmemBytes);
    if (e != cudaSuccess) return e;
    const int n_pairs = ((s.Skv + kTile - 1) / kTile + 1) / 2;  // a CTA works through two key tiles
    e = launch_dependent(nk, dim3(static_cast<unsigned>(n_pairs) * p.n_qchunks * s.B * s.H), dim3(kThreads), kNzSmemBytes,
                         stream, mq, mk, mn, p);
    count_launch();
  } else
#endif
  {
  const int n_kvb = (s.Skv + 2 * kTile - 1) / (2 * kTile);
  const dim3 grid(static_cast<unsigned>(n_kvb) * p.n_qchunks * s.B * s.H);
  void (*kern)(CUtensorMap, CUtensorMap, ColParams) = nullptr;
  if (a.mode == ASUKA_SCORE_SUM) kern = s.bf16 ? col_scores_kernel<true, 0> : col_scores_kernel<false, 0>;
  else if (a.mode == ASUKA_SCORE_SUM_SQ) kern = s.bf16 ? col_scores_kernel<true, 1> : col_scores_kernel<false, 1>;
  else if (a.mode == ASUKA_SCORE_CORM) kern = s.bf16 ? col_scores_kernel<true, 4> : col_scores_kernel<false, 4>;
  else if (a.exp_rand != nullptr) kern = s.bf16 ? col_scores_kernel<true, 2> : col_scores_kernel<false, 2>;
  else kern = s.bf16 ? col_scores_kernel<true, 3> : col_scores_kernel<false, 3>;
  e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (e != cudaSuccess) return e;
  e = launch_dependent(kern, grid, dim3(kThreads), kSmemBytes, stream, mq, mk, p);
  count_launch();
  }
  if (e != cudaSuccess || p.n_qchunks == 1) return e;
  const size_t n = static_cast<size_t>(s.B) * s.H * s.Skv;
  const bool sq = a.mode == ASUKA_SCORE_SUM_SQ;
  if (pending != nullptr) {  // the caller's next kernel adds the partial sums
    pending->part = p.part;
    pending->part_sq = sq ? p.part_sq : nullptr;
    pending->n_chunks = p.n_qchunks;
    return e;
  }
  e = launch_dependent(sum_chunks_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, stream,
                       static_cast<const float*>(p.part), static_cast<const float*>(sq ? p.part_sq : nullptr),
                       a.score, a.score_sq, p.n_qchunks, n);
  count_launch();
  return e;
}

cudaError_t launch_kf_rowstat(const CUtensorMap& mq, const CUtensorMap& mk, const ScoreArgs& a,
                              float* lse2_out, const AttnShape& s, cudaStream_t stream) {
  const ColParams p = make_params(a, s);
  const dim3 grid(static_cast<unsigned>(p.nq_tiles) * s.B * s.H);
  cudaError_t e;
  if (a.exp_rand == nullptr) {
    auto kern = s.bf16 ? kf_rowstat_kernel<true, 2> : kf_rowstat_kernel<false, 2>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), RsCfg<2>::kSmem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kRsThreads, RsCfg<2>::kSmem, stream>>>(mq, mk, mq, p, lse2_out);
    count_launch();
    return cudaGetLastError();
  }
  // TMA needs a 16-byte aligned base and strides that are multiples of 16 bytes
  const bool tma_ok = (reinterpret_cast<uintptr_t>(a.exp_rand) & 15u) == 0 && a.er_stride_q % 4 == 0 &&
                      a.er_stride_h % 4 == 0 && a.er_stride_b % 4 == 0 && a.er_stride_q > 0 &&
                      a.er_stride_h > 0 && a.er_stride_b > 0;
  if (tma_ok) {
    CUtensorMap mn;
    const uint64_t dims[4] = {static_cast<uint64_t>(s.Skv), static_cast<uint64_t>(s.Sq),
                              static_cast<uint64_t>(s.H), static_cast<uint64_t>(s.B)};
    const uint64_t strides[3] = {static_cast<uint64_t>(a.er_stride_q) * 4, static_cast<uint64_t>(a.er_stride_h) * 4,
                                 static_cast<uint64_t>(a.er_stride_b) * 4};
    const uint32_t box[4] = {32, 128, 1, 1};
    if (tma_host::make_f32_map_sw128(&mn, a.exp_rand, dims, strides, box) != 0) return cudaErrorInvalidValue;
    auto kern = s.bf16 ? kf_rowstat_kernel<true, 1> : kf_rowstat_kernel<false, 1>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), RsCfg<1>::kSmem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kRsThreads, RsCfg<1>::kSmem, stream>>>(mq, mk, mn, p, lse2_out);
  } else {
    auto kern = s.bf16 ? kf_rowstat_kernel<true, 0> : kf_rowstat_kernel<false, 0>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), RsCfg<0>::kSmem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kRsThreads, RsCfg<0>::kSmem, stream>>>(mq, mk, mq, p, lse2_out);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace asuka
