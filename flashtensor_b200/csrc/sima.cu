// SimA softmax-free attention for sm_100a:
//   Qn = Q / sum_s |Q|,  Kn = K / sum_s |K|  (per channel, over the sequence; no epsilon),
//   out = Qn (Kn^T V), non-causal.
// Replaces the kernels the Asuka pipeline generates for bench/sima.mlir:13-17, with the L1
// normalisation of lib/Dialect/Asuka/Transforms/LowerComplexReduce.cpp:44-69.
//
// Algebra: out[s,e] = sum_d Q[s,d] * M'[d,e] with M'[d,e] = (sum_s K[s,d] V[s,e]) / (ck[d] cq[d]),
// so the sequence is streamed twice and no S x S tensor exists:
//   1. sima_stats_kernel   every CTA streams a slab of the sequence of one (batch, head): K^T V on
//                          tcgen05 (both operands MN-major straight from the TMA tiles), and the
//                          column sums of |K| and |Q| with 128-bit shared-memory loads.  Partial
//                          results go to the workspace.
//   2. sima_reduce_kernel  sums the partials in a fixed order, divides by ck*cq, and writes M'^T in
//                          the 16-bit input type scaled by a power of two per block of 32 output
//                          channels (the entries are ~1e-6, far below fp16's normal range), plus
//                          the inverse scales.
//   3. sima_out_kernel     streams Q again: out = (Q M'') * inverse scale, tcgen05 with the
//                          accumulator double-buffered in TMEM, TMA store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace asuka {
using namespace sm100;

namespace {

constexpr int kTile = 128;
constexpr uint32_t kTileBytes = 128 * 128 * 2;
constexpr uint32_t kHalfBytes = kTileBytes / 2;
constexpr int kMElems = 128 * 128;

__device__ __forceinline__ void record_timeout(uint32_t* status, uint32_t site) {
  atomicAdd(&status[0], 1u);
  status[1] = site;
}

struct SimaWs {
  float* part_m;     // [BH][nchunks][e][d]  partial (K^T V)^T
  float* part_c;     // [BH][nchunks][2][128] partial ck, cq
  uint16_t* m16;     // [BH][e][d] scaled M'^T in the input type
  float* inv_scale;  // [BH][4]: one per block of 32 output channels
};

// ---------------------------------------------------------------------------------------------
// 1. statistics: partial K^T V, sum|K|, sum|Q| over a slab of the sequence
// ---------------------------------------------------------------------------------------------
constexpr int kStThreads = 384;
constexpr int kStStages = 2;
constexpr uint32_t kStSmem = kStStages * 3 * kTileBytes + 1024;

struct StatsParams {
  int B, H, S;
  int nchunks, tiles_per_chunk, ntiles;
  int ea;            // 1: the EA program (softmax normalisations), 0: SimA (L1 normalisations)
  SimaWs ws;
  uint32_t* status;
};

struct StBars {
  uint64_t full[3], empty[3], m_done;  // (two stages in SimA mode, three in EA mode)
  uint64_t ktrans[3];                  // EA only: the K tile of the stage has been exponentiated in place
};

template <bool kBF16>
__device__ __forceinline__ void abs_acc8(const uint4& v, float (&acc)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f;
    if constexpr (kBF16) {
      f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    } else {
      f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    acc[2 * i] += fabsf(f.x);
    acc[2 * i + 1] += fabsf(f.y);
  }
}

template <bool kBF16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t;
    if constexpr (kBF16) {
      t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    } else {
      t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
// rounds to the 16-bit type; `f` is overwritten with the rounded values
template <bool kBF16>
__device__ __forceinline__ uint4 pack8(float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (kBF16) {
      __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
      const float2 r = __bfloat1622float2(t);
      f[2 * i] = r.x;
      f[2 * i + 1] = r.y;
    } else {
      __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
      const float2 r = __half22float2(t);
      f[2 * i] = r.x;
      f[2 * i + 1] = r.y;
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <bool kBF16>
__device__ __forceinline__ float2 unpack2_16(uint32_t w) {
  if constexpr (kBF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool kBF16>
__device__ __forceinline__ uint32_t pack2_16(float2 f) {
  if constexpr (kBF16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(f.x, f.y);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}
// element-wise maximum of two packed pairs of 16-bit values
template <bool kBF16>
__device__ __forceinline__ uint32_t max2_16(uint32_t a, uint32_t b) {
  if constexpr (kBF16) {
    __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
// true if either element of the packed pair a exceeds the matching element of b
template <bool kBF16>
__device__ __forceinline__ bool any_gt2_16(uint32_t a, uint32_t b) {
  if constexpr (kBF16) {
    const __nv_bfloat162 r = __hgt2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r) != 0u;
  } else {
    const __half2 r = __hgt2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r) != 0u;
  }
}
// EA: how far (natural-log units) a value of K may exceed its column's reference before the
// reference is raised; exp(8) = 2981 is far inside the range of both 16-bit types
constexpr float kEaSlack = 8.0f;
// EA: of the four pairs of exponentials per 16-byte chunk, how many go to the FMA pipe
#ifndef ASUKA_EA_POLY_PAIRS
#define ASUKA_EA_POLY_PAIRS 0
#endif
constexpr int kEaPolyPairs = ASUKA_EA_POLY_PAIRS;
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kEA: the EA program (softmax over the sequence of k, bench/ea.mlir:14).  K is exponentiated in
// place in shared memory against a per-column reference of the slab before the MMA reads it, so
// the product is exp(K - ref)^T V; the column sums of the same rounded values (a second, 16-column
// MMA against a block of ones) are the slab's part of the softmax denominators.  The reduce brings
// the slabs to a common reference.  Q is not needed in this pass.
template <bool kBF16, bool kEA>
__global__ void __launch_bounds__(kStThreads, 1)
sima_stats_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const StatsParams p) {
  // EA does not read Q in this pass: the same shared memory then holds three stages of [K | V]
  // instead of two of [K | V | Q], i.e. two stages instead of one in flight while one is consumed
  constexpr int kSt = kEA ? 3 : 2;
  constexpr uint32_t kStageBytes = (kEA ? 2 : 3) * kTileBytes;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) StBars bars;
  __shared__ float red[2][8][kTile];
  __shared__ float ref_s[kTile];
  // EA: a block of ones, the B operand of the small MMA that gives the column sums of the
  // exponentiated K (every element is 1, so its layout does not matter)
  __shared__ __align__(1024) uint16_t ones_s[kEA ? 1024 : 8];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;
  const int chunk = static_cast<int>(blockIdx.x) % p.nchunks;
  const int bh = static_cast<int>(blockIdx.x) / p.nchunks;
  const int b = bh / p.H, h = bh % p.H;
  const int tile0 = chunk * p.tiles_per_chunk;
  const int ntile = max(0, min(p.tiles_per_chunk, p.ntiles - tile0));

  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < kSt; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), 1 + 8);
    }
    mbar_init(smem_u32(&bars.m_done), 1);
    for (int i = 0; i < kSt; ++i) mbar_init(smem_u32(&bars.ktrans[i]), 256);
    mbar_fence_init();
  }
  if constexpr (kEA) {
    for (int i = tid; i < 1024; i += kStThreads) ones_s[i] = kBF16 ? 0x3F80 : 0x3C00;
    fence_proxy_async_smem();
  }
  constexpr uint32_t kTmemCols = kEA ? 256 : 128;  // EA: columns 128.. hold the column sums
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;

  // stage layout: [K | V | Q] tiles
  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < ntile; ++i) {
        const int k = i;
        const int st = k % kSt;
        if (k >= kSt && !mbar_wait(smem_u32(&bars.empty[st]), (k / kSt - 1) & 1, abortp)) {
          record_timeout(p.status, 41);
          break;
        }
        const uint32_t bar = smem_u32(&bars.full[st]);
        const uint32_t base = smem_base + st * kStageBytes;
        const int s0 = (tile0 + i) * kTile;
        mbar_expect_tx(bar, (kEA ? 2 : 3) * kTileBytes);
        if constexpr (kEA) {
          const uint64_t drop = l2_policy_evict_first();
          tma_load_4d_hint(base, &map_k, bar, 0, h, s0, b, drop);
          tma_load_4d_hint(base + kHalfBytes, &map_k, bar, 64, h, s0, b, drop);
          tma_load_4d_hint(base + kTileBytes, &map_v, bar, 0, h, s0, b, drop);
          tma_load_4d_hint(base + kTileBytes + kHalfBytes, &map_v, bar, 64, h, s0, b, drop);
        } else {
          tma_load_4d(base, &map_k, bar, 0, h, s0, b);
          tma_load_4d(base + kHalfBytes, &map_k, bar, 64, h, s0, b);
          tma_load_4d(base + kTileBytes, &map_v, bar, 0, h, s0, b);
          tma_load_4d(base + kTileBytes + kHalfBytes, &map_v, bar, 64, h, s0, b);
        }
        if constexpr (!kEA) {
          tma_load_4d(base + 2 * kTileBytes, &map_q, bar, 0, h, s0, b);
          tma_load_4d(base + 2 * kTileBytes + kHalfBytes, &map_q, bar, 64, h, s0, b);
        }
      }
    }
  } else if (warp == 1) {
    // whole warp walks the loop; one elected lane issues the MMAs
    {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_MN_MAJOR, UMMA_MN_MAJOR, 128, 128);
      bool ok = true;
      for (int i = 0; i < ntile && ok; ++i) {
        const int k = i;
        const int st = k % kSt;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[st]), (k / kSt) & 1, abortp));
        if (!ok) { if (lane == 0) record_timeout(p.status, 42); break; }
        if constexpr (kEA) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.ktrans[i % kSt]), (i / kSt) & 1, abortp));
          if (!ok) { if (lane == 0) record_timeout(p.status, 45); break; }
        }
        tc_fence_after_sync();
        const uint32_t base = smem_base + st * kStageBytes;
        // M = K^T V: TMEM lane = d, column = e
        const uint64_t adesc = umma_smem_desc_sw128(base, kHalfBytes, 1024);               // K
        const uint64_t bdesc = umma_smem_desc_sw128(base + kTileBytes, kHalfBytes, 1024);  // V
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>(kk * (2048 >> 4));
            umma_ss(tbase, adesc + off, bdesc + off, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
          if constexpr (kEA) {
            // column sums of the exponentiated (and rounded) K: the same A against 16 columns of ones
            constexpr uint32_t idesc16 = umma_idesc_f16(kFmt, UMMA_MN_MAJOR, UMMA_MN_MAJOR, 128, 16);
            const uint64_t odesc = umma_smem_desc_sw128(smem_u32(ones_s), 1024, 1024);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t off = static_cast<uint64_t>(kk * (2048 >> 4));
              umma_ss(tbase + 128, adesc + off, odesc, idesc16, (i > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&bars.empty[st]));
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(smem_u32(&bars.m_done));
      __syncwarp();
    }
  } else if (warp >= 4) {
    // warps 4-7: |K| column sums; warps 8-11: |Q| column sums
    const int which = (warp - 4) >> 2;  // 0 = K, 1 = Q
    const int t128 = tid - 128 - which * 128;
    const int chunk16 = t128 & 15;   // 8 consecutive channels
    const int rg = t128 >> 4;        // rows rg, rg+8, ...
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    if constexpr (kEA) {
      // All 256 threads work on the K tile, rows 16 apart per thread: k' = exp(k - ref), rounded to
      // the input type and written back for the MMA; rows past the sequence give 0.  `ref` is a
      // per-column reference for the whole slab (the reduce brings the slabs to a common one): the
      // column maxima of the slab's first tile, raised -- with the accumulators scaled to match --
      // whenever a later value exceeds it by more than kEaSlack, so that k' stays far inside the
      // range of the 16-bit type.  On ordinary data the raise never happens after the first tile.
      const int wq = warp & 3;
      const int rg16 = which * 8 + rg;
      const float kL2e = 1.4426950408889634f;
      float2 nref[4] = {};   // -ref * log2(e) of this thread's eight channels
      uint32_t thr[4] = {};  // ref + kEaSlack in the input type, packed
      bool dead = false;     // a wait has given up: no more work, but every barrier is still taken
      for (int i = 0; i < ntile; ++i) {
        const int st = i % kSt;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[st]), (i / kSt) & 1, abortp))) {
          if (lane == 0 && !dead) record_timeout(p.status, 43);
          dead = true;
        }
        uint8_t* tile = smem_gen + st * kStageBytes + (chunk16 >> 3) * kHalfBytes;
        const int s0 = (tile0 + i) * kTile;
        uint4 raw[8];
        uint32_t m4[4];  // maxima over this thread's rows, packed as loaded (exact for 16-bit values)
#pragma unroll
        for (int e = 0; e < 4; ++e) m4[e] = kBF16 ? 0xFF80FF80u : 0xFC00FC00u;  // -inf, -inf
        if (!dead) {
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int row = rg16 + 16 * r;
            raw[r] = *reinterpret_cast<const uint4*>(tile + sw128_offset(row, chunk16 & 7));
            if (s0 + row < p.S) {  // (rows past the sequence were zero-filled by the load)
              m4[0] = max2_16<kBF16>(m4[0], raw[r].x);
              m4[1] = max2_16<kBF16>(m4[1], raw[r].y);
              m4[2] = max2_16<kBF16>(m4[2], raw[r].z);
              m4[3] = max2_16<kBF16>(m4[3], raw[r].w);
            }
          }
        }
        bool raise = i == 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) raise = raise || any_gt2_16<kBF16>(m4[e], thr[e]);
        if (named_bar_or(1, 256, raise && !dead)) {
          float mx[8];
          unpack8<kBF16>(make_uint4(m4[0], m4[1], m4[2], m4[3]), mx);
#pragma unroll
          for (int e = 0; e < 8; ++e) red[which][rg][chunk16 * 8 + e] = mx[e];
          named_bar_sync(1, 256);
          if (which == 0) {  // thread t128 = column d = TMEM lane d
            float tmax = -INFINITY;
#pragma unroll
            for (int g = 0; g < 8; ++g) tmax = fmaxf(tmax, fmaxf(red[0][g][t128], red[1][g][t128]));
            const float old = ref_s[t128];
            const float nw = i == 0 ? tmax : fmaxf(old, tmax);
            ref_s[t128] = nw;
            if (i > 0) {
              // every MMA issued so far has retired once the release of the previous tile's stage
              // has fired (the MMA of this tile waits for the arrivals below)
              if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.empty[(i - 1) % kSt]), ((i - 1) / kSt) & 1, abortp))) {
                if (lane == 0 && !dead) record_timeout(p.status, 46);
                dead = true;
              }
              if (!dead) {
                tc_fence_after_sync();
                const float f = nw > old ? ex2_approx((old - nw) * kL2e) : 1.f;
                const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  uint32_t u[32];
                  tmem_ld32(tbase + lane_base + c * 32, u);
                  tmem_wait_ld();
#pragma unroll
                  for (int x = 0; x < 32; ++x) u[x] = __float_as_uint(__uint_as_float(u[x]) * f);
                  tmem_st32(tbase + lane_base + c * 32, u);
                }
                uint32_t u[16];
                tmem_ld16(tbase + lane_base + 128, u);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 16; ++x) u[x] = __float_as_uint(__uint_as_float(u[x]) * f);
                tmem_st16(tbase + lane_base + 128, u);
                tmem_wait_st();
                tc_fence_before_sync();
              }
            }
          }
          named_bar_sync(1, 256);  // references updated, accumulators scaled
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float r0 = ref_s[chunk16 * 8 + 2 * e], r1 = ref_s[chunk16 * 8 + 2 * e + 1];
            nref[e] = make_float2(-r0 * kL2e, -r1 * kL2e);
            thr[e] = pack2_16<kBF16>(make_float2(r0 + kEaSlack, r1 + kEaSlack));
          }
          dead = dead || *abortp != 0u;
        }
        if (!dead) {
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int row = rg16 + 16 * r;
            uint4* ptr = reinterpret_cast<uint4*>(tile + sw128_offset(row, chunk16 & 7));
            if (s0 + row < p.S) {
              const uint32_t w[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 x = __ffma2_rn(unpack2_16<kBF16>(w[e]), make_float2(kL2e, kL2e), nref[e]);
                const float2 y = e < kEaPolyPairs ? ex2_fma_pipe2(x) : make_float2(ex2_approx(x.x), ex2_approx(x.y));
                o[e] = pack2_16<kBF16>(y);
              }
              *ptr = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
              *ptr = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          fence_proxy_async_smem();  // written by ordinary stores, read by the tensor pipe
          mbar_arrive(smem_u32(&bars.ktrans[st]));
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.empty[st]));
        }
      }
      ok = !dead;
    } else {
      for (int i = 0; i < ntile; ++i) {
        const int st = i % kSt;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[st]), (i / kSt) & 1, abortp));
        if (!ok) { if (lane == 0) record_timeout(p.status, 43); break; }
        const uint8_t* tile = smem_gen + st * kStageBytes + (which ? 2 * kTileBytes : 0) +
                              (chunk16 >> 3) * kHalfBytes;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const int row = rg + 8 * r;
          const uint4 v = *reinterpret_cast<const uint4*>(tile + sw128_offset(row, chunk16 & 7));
          abs_acc8<kBF16>(v, acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.empty[st]));
      }
    }
    if constexpr (kEA) {
      // slot 1 of the partial (SimA's sum|Q|): the slab's per-column reference; slot 0 is written below
      if (which == 1)
        p.ws.part_c[((static_cast<size_t>(bh) * p.nchunks + chunk) * 2 + 1) * kTile + t128] = ref_s[t128];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) red[which][rg][chunk16 * 8 + i] = acc[i];
      named_bar_sync(1 + which, 128);
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) s += red[which][g][t128];
      p.ws.part_c[((static_cast<size_t>(bh) * p.nchunks + chunk) * 2 + which) * kTile + t128] = s;
    }
    if (which == 0) {
      // warps 4-7 also drain the accumulator: lane = d, column = e
      float* dst = p.ws.part_m + (static_cast<size_t>(bh) * p.nchunks + chunk) * kMElems;
      const int wq = warp & 3;
      const int d = wq * 32 + lane;
      if (ntile > 0) {
        ok = ok && __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.m_done), 0, abortp));
        if (ok) {
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t u[32];
            tmem_ld32(tbase + (static_cast<uint32_t>(wq * 32) << 16) + c * 32, u);
            tmem_wait_ld();
            // thread d holds M[d][e..]; element (d, e) -> dst[e * 128 + d]: consecutive threads
            // hit consecutive addresses and the partial is stored transposed, [e][d]
#pragma unroll
            for (int i = 0; i < 32; ++i) dst[(c * 32 + i) * kTile + d] = __uint_as_float(u[i]);
          }
          if constexpr (kEA) {
            // slot 0: this slab's part of the softmax denominators (relative to the slab's maxima)
            uint32_t u[16];
            tmem_ld16(tbase + (static_cast<uint32_t>(wq * 32) << 16) + 128, u);
            tmem_wait_ld();
            p.ws.part_c[((static_cast<size_t>(bh) * p.nchunks + chunk) * 2 + 0) * kTile + d] = __uint_as_float(u[0]);
          }
        } else if (lane == 0) {
          record_timeout(p.status, 44);
        }
      } else {
        for (int i = 0; i < 128; ++i) dst[i * kTile + d] = 0.f;
        if constexpr (kEA) p.ws.part_c[((static_cast<size_t>(bh) * p.nchunks + chunk) * 2 + 0) * kTile + d] = 0.f;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// 2. reduce partials, normalise, scale into the 16-bit type.  part_m and the output m16 are
//    both stored [e][d] (d contiguous): the K-major B operand of step 3.
// ---------------------------------------------------------------------------------------------
// One CTA per (head, block of 32 output channels e): 4096 entries of M'^T, its own power-of-two
// scale (the epilogue of step 3 multiplies each 32-column chunk by the matching inverse).
constexpr int kRedBlocks = 4;
constexpr int kMaxChunks = 16;  // slabs per (batch, head) in the three-kernel path
constexpr int kRedElems = kMElems / kRedBlocks;
template <bool kBF16>
__global__ void __launch_bounds__(256, 4) sima_reduce_kernel(const StatsParams p) {
  __shared__ float inv_c[kTile];
  __shared__ float w_s[kMaxChunks][kTile];  // EA: exp(slab reference - largest reference), per slab and column
  __shared__ float wmax[8];
  __shared__ float s_scale;
  const int blk = blockIdx.x % kRedBlocks;
  const int bh = blockIdx.x / kRedBlocks, tid = threadIdx.x;
  const float* pc = p.ws.part_c + static_cast<size_t>(bh) * p.nchunks * 2 * kTile;
  const float* pm = p.ws.part_m + static_cast<size_t>(bh) * p.nchunks * kMElems + blk * kRedElems;
  if (tid < kTile) {
    if (p.ea) {
      // each slab's exponentials were taken against the slab's own per-column reference (slot 1):
      // bring them to the largest of these
      float m = -INFINITY;
      for (int c = 0; c < p.nchunks; ++c) m = fmaxf(m, pc[(c * 2 + 1) * kTile + tid]);
      float ck = 0.f;
      for (int c = 0; c < p.nchunks; ++c) {
        const float w = __expf(pc[(c * 2 + 1) * kTile + tid] - m);
        w_s[c][tid] = w;
        ck = fmaf(pc[(c * 2 + 0) * kTile + tid], w, ck);
      }
      inv_c[tid] = __fdiv_rn(1.0f, ck);
    } else {
      float ck = 0.f, cq = 0.f;
      for (int c = 0; c < p.nchunks; ++c) {
        ck += pc[(c * 2 + 0) * kTile + tid];
        cq += pc[(c * 2 + 1) * kTile + tid];
      }
      inv_c[tid] = __fdiv_rn(1.0f, __fmul_rn(ck, cq));
    }
  }
  __syncthreads();
  float vals[kRedElems / 256];
  float amax = 0.f;
#pragma unroll
  for (int it = 0; it < kRedElems / 256; ++it) {
    const int idx = it * 256 + tid;  // = e_local * 128 + d
    float m = 0.f;
    if (p.ea) {
      for (int c = 0; c < p.nchunks; ++c) m = fmaf(pm[static_cast<size_t>(c) * kMElems + idx], w_s[c][idx & 127], m);
    } else {
      for (int c = 0; c < p.nchunks; ++c) m += pm[static_cast<size_t>(c) * kMElems + idx];
    }
    m *= inv_c[idx & 127];
    vals[it] = m;
    amax = fmaxf(amax, fabsf(m));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((tid & 31) == 0) wmax[tid >> 5] = amax;
  __syncthreads();
  if (tid == 0) {
    float a = 0.f;
    for (int i = 0; i < 8; ++i) a = fmaxf(a, wmax[i]);
    float sc = 1.f;
    if (a > 0.f && a < INFINITY) {
      int ex;
      frexpf(a, &ex);            // a = f * 2^ex, f in [0.5, 1)
      sc = ldexpf(1.0f, 14 - ex);  // a * sc in [2^13, 2^14)
    }
    s_scale = sc;
    p.ws.inv_scale[bh * kRedBlocks + blk] = 1.0f / sc;
  }
  __syncthreads();
  const float sc = s_scale;
  uint16_t* dst = p.ws.m16 + static_cast<size_t>(bh) * kMElems + blk * kRedElems;
#pragma unroll
  for (int it = 0; it < kRedElems / 256; ++it) {
    const int idx = it * 256 + tid;
    const float v = vals[it] * sc;
    uint16_t bits;
    if constexpr (kBF16) {
      __nv_bfloat16 hb = __float2bfloat16_rn(v);
      bits = *reinterpret_cast<uint16_t*>(&hb);
    } else {
      __half hh = __float2half_rn(v);
      bits = *reinterpret_cast<uint16_t*>(&hh);
    }
    dst[idx] = bits;
  }
}

// ---------------------------------------------------------------------------------------------
// 3. out = (Q M'') * inv_scale
// ---------------------------------------------------------------------------------------------
constexpr int kOutThreads = 256;  // warp 0 producer, warp 1 MMA, warp 2 stores (16-bit output), warps 4-7 epilogue
// Q stages.  16-bit output: the epilogue writes a tile's result over the Q tile it came from (the
// MMA has consumed it by then) and the stage goes back to the producer once the store has read it,
// so all of shared memory beside M'' is one ring of stages.  f32 output: a 64 KB staging buffer.
__host__ __device__ constexpr int out_stages(bool out_f32, bool ea) { return out_f32 ? (ea ? 3 : 4) : (ea ? 5 : 6); }
__host__ __device__ constexpr uint32_t out_smem_bytes(bool out_f32, bool ea) {
  return (1 + out_stages(out_f32, ea) + (out_f32 ? 2 : 0)) * kTileBytes + 1024;
}

struct OutParams {
  int B, H, S;
  int ntiles, tiles_per_cta, nqchunks;
  const float* inv_scale;
  float* out_f32;  // non-null selects the f32 output path
  int64_t o_sb, o_ss, o_sh;
  uint32_t* status;
};

struct OutBars {
  uint64_t m_full, q_full[6], q_empty[6], acc_full[2], acc_empty[2];
  uint64_t qtrans[6];     // EA only: the Q tile of the stage has been exponentiated in place
  uint64_t out_ready[6];  // 16-bit output: the result tile has been written into the stage
};

// kEA: softmax over the features of every query row (bench/ea.mlir:13): eight more warps
// exponentiate the Q tile in place in shared memory against the row maxima before the MMA reads
// it; a second, 16-column MMA against a block of ones gives the row sums of exactly the rounded
// values the first one multiplies, and the epilogue divides by them.
template <bool kBF16, bool kOutF32, bool kEA>
__global__ void __launch_bounds__(kOutThreads + (kEA ? 256 : 0), 1)  // EA: warps 8-15 exponentiate Q
sima_out_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_m,
                const __grid_constant__ CUtensorMap map_o, const OutParams p) {
  constexpr int kQ = out_stages(kOutF32, kEA);
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) OutBars bars;
  // EA: a block of ones, the B operand of the small MMA that gives the row sums of the
  // exponentiated Q (every element is 1, so its layout does not matter)
  __shared__ __align__(1024) uint16_t ones_s[kEA ? 1024 : 8];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sM = smem_base;
  const uint32_t sQ = smem_base + kTileBytes;
  const uint32_t sO = sQ + kQ * kTileBytes;  // f32 output only: one 64 KB staging buffer

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;
  const int qc = static_cast<int>(blockIdx.x) % p.nqchunks;
  const int bh = static_cast<int>(blockIdx.x) / p.nqchunks;
  const int b = bh / p.H, h = bh % p.H;
  const int tile0 = qc * p.tiles_per_cta;
  const int ntile = max(0, min(p.tiles_per_cta, p.ntiles - tile0));

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&bars.m_full), 1);
    for (int i = 0; i < kQ; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.acc_full[i]), 1);
      mbar_init(smem_u32(&bars.acc_empty[i]), 128);
    }
    for (int i = 0; i < kQ; ++i) {
      mbar_init(smem_u32(&bars.qtrans[i]), 256);
      mbar_init(smem_u32(&bars.out_ready[i]), 128);
    }
    mbar_fence_init();
  }
  if constexpr (kEA) {
    for (int i = tid; i < 1024; i += kOutThreads + 256) ones_s[i] = kBF16 ? 0x3F80 : 0x3C00;
    fence_proxy_async_smem();
  }
  // two accumulators of 128 columns; EA: columns 256.. and 272.. hold the row sums of the two
  constexpr uint32_t kTmemCols = kEA ? 512 : 256;
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;

  if (warp == 0) {
    if (lane == 0 && ntile > 0) {
      {
        const uint32_t bar = smem_u32(&bars.m_full);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sM, &map_m, bar, 0, 0, bh * kTile, 0);
        tma_load_4d(sM + kHalfBytes, &map_m, bar, 64, 0, bh * kTile, 0);
      }
      for (int i = 0; i < ntile; ++i) {
        const int st = i % kQ;
        const uint32_t use = static_cast<uint32_t>(i / kQ);
        if (use > 0 && !mbar_wait(smem_u32(&bars.q_empty[st]), (use - 1) & 1, abortp)) {
          record_timeout(p.status, 51);
          break;
        }
        const uint32_t bar = smem_u32(&bars.q_full[st]);
        mbar_expect_tx(bar, kTileBytes);
        tma_load_4d(sQ + st * kTileBytes, &map_q, bar, 0, h, (tile0 + i) * kTile, b);
        tma_load_4d(sQ + st * kTileBytes + kHalfBytes, &map_q, bar, 64, h, (tile0 + i) * kTile, b);
      }
    }
  } else if (warp == 1) {
    if (ntile > 0) {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
        const bool good = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, abortp));
        if (!good && lane == 0) record_timeout(p.status, site);
        return good;
      };
      bool ok = wait_all(&bars.m_full, 0, 52);
      const uint64_t mdesc = umma_smem_desc_sw128(sM, 16, 1024);
      for (int i = 0; i < ntile && ok; ++i) {
        const int st = i % kQ, buf = i & 1;
        ok = wait_all(&bars.q_full[st], (i / kQ) & 1, 53);
        if (!ok) break;
        if constexpr (kEA) {
          ok = wait_all(&bars.qtrans[st], (i / kQ) & 1, 56);
          if (!ok) break;
        }
        if (i >= 2) {
          ok = wait_all(&bars.acc_empty[buf], ((i >> 1) - 1) & 1, 54);
          if (!ok) break;
        }
        tc_fence_after_sync();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ + st * kTileBytes, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
            umma_ss(tbase + buf * 128, qdesc + off, mdesc + off, idesc, kk > 0 ? 1u : 0u);
          }
          if constexpr (kEA) {
            // row sums of the exponentiated (and rounded) Q: the same A against 16 columns of ones
            constexpr uint32_t idesc16 = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 16);
            const uint64_t odesc = umma_smem_desc_sw128(smem_u32(ones_s), 1024, 1024);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
              umma_ss(tbase + 256 + buf * 16, qdesc + off, odesc, idesc16, kk > 0 ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&bars.acc_full[buf]));
          if constexpr (kOutF32) umma_commit(smem_u32(&bars.q_empty[st]));  // (else: the store warp releases it)
        }
        __syncwarp();
      }
    }
  } else if (!kOutF32 && warp == 2) {
    // ---------------------------------------------------------------- 16-bit output: store warp
    if (lane == 0) {
      for (int i = 0; i < ntile; ++i) {
        const int st = i % kQ;
        if (!mbar_wait(smem_u32(&bars.out_ready[st]), (i / kQ) & 1, abortp)) {
          record_timeout(p.status, 58);
          break;
        }
        const int s0 = (tile0 + i) * kTile;
        tma_store_4d(&map_o, sQ + st * kTileBytes, 0, h, s0, b);
        tma_store_4d(&map_o, sQ + st * kTileBytes + kHalfBytes, 64, h, s0, b);
        tma_store_commit();
        tma_store_wait_read();  // the stage may be overwritten from here on
        mbar_arrive(smem_u32(&bars.q_empty[st]));
      }
      tma_store_wait_all();
    }
  } else if (kEA && warp >= 8) {
    // ------------------------------------------------------------- EA: softmax numerators of Q
    // Two threads per row (adjacent lanes, 64 features each) exponentiate every Q tile in place
    // against the row maximum; the row sums come from the tensor pipe (above).  Half of the
    // exponentials run on the special-function unit, half on the FMA pipe.
    const int t256 = tid - 256;
    const int r = t256 >> 1, half = t256 & 1;
    const float kL2e = 1.4426950408889634f;
    bool ok = true;
    for (int i = 0; i < ntile && ok; ++i) {
      const int st = i % kQ;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.q_full[st]), (i / kQ) & 1, abortp));
      if (!ok) { if (lane == 0) record_timeout(p.status, 57); break; }
      uint8_t* tile = smem_gen + (sQ - smem_base) + st * kTileBytes + half * kHalfBytes;
      uint4 raw[8];
      uint32_t mxp = kBF16 ? 0xFF80FF80u : 0xFC00FC00u;  // (-inf, -inf); the maximum of 16-bit values is exact
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        raw[c] = *reinterpret_cast<const uint4*>(tile + sw128_offset(r, c));
        mxp = max2_16<kBF16>(mxp, max2_16<kBF16>(max2_16<kBF16>(raw[c].x, raw[c].y), max2_16<kBF16>(raw[c].z, raw[c].w)));
      }
      const float2 m2 = unpack2_16<kBF16>(mxp);
      float mx = fmaxf(m2.x, m2.y);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      const float2 neg = make_float2(-mx * kL2e, -mx * kL2e);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __ffma2_rn(unpack2_16<kBF16>(w[e]), make_float2(kL2e, kL2e), neg);
          const float2 y = e < kEaPolyPairs ? ex2_fma_pipe2(x) : make_float2(ex2_approx(x.x), ex2_approx(x.y));
          o[e] = pack2_16<kBF16>(y);
        }
        *reinterpret_cast<uint4*>(tile + sw128_offset(r, c)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();  // the tile was written by ordinary stores, the tensor pipe reads it
      mbar_arrive(smem_u32(&bars.qtrans[st]));
    }
  } else if (warp >= 4 && warp < 8) {
    const int wq = warp & 3;
    const int r = wq * 32 + lane;  // row of the tile
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    // one inverse scale per block of 32 output channels = per TMEM chunk below
    const float inv4[4] = {p.inv_scale[bh * 4 + 0], p.inv_scale[bh * 4 + 1], p.inv_scale[bh * 4 + 2],
                           p.inv_scale[bh * 4 + 3]};
    bool ok = true;
    for (int i = 0; i < ntile && ok; ++i) {
      const int buf = i & 1;
      const int s0 = (tile0 + i) * kTile;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_full[buf]), (i >> 1) & 1, abortp));
      if (!ok) { if (lane == 0) record_timeout(p.status, 55); break; }
      tc_fence_after_sync();
      float inv_r = 1.f;
      if constexpr (kEA) {
        uint32_t u[16];
        tmem_ld16(tbase + lane_base + 256 + buf * 16, u);
        tmem_wait_ld();
        inv_r = 1.f / __uint_as_float(u[0]);
      }
      // f32: the staging buffer is free again once the previous tile's copy-out has passed the
      // barrier; 16-bit: the result goes over the Q tile of this stage, which the MMA has consumed
      if constexpr (kOutF32) named_bar_sync(1, 128);
      uint8_t* stage = smem_gen + (kOutF32 ? (sO - smem_base) : (sQ - smem_base) + (i % kQ) * kTileBytes);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t u[32];
        tmem_ld32(tbase + lane_base + buf * 128 + c * 32, u);
        tmem_wait_ld();
        const float inv_sc = kEA ? inv4[c] * inv_r : inv4[c];
        if constexpr (kOutF32) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 v;
            v.x = __uint_as_float(u[g * 4 + 0]) * inv_sc;
            v.y = __uint_as_float(u[g * 4 + 1]) * inv_sc;
            v.z = __uint_as_float(u[g * 4 + 2]) * inv_sc;
            v.w = __uint_as_float(u[g * 4 + 3]) * inv_sc;
            const int chunk = c * 8 + g;  // 16-byte chunk of the 512-byte row
            *reinterpret_cast<float4*>(stage + r * 512 + ((chunk ^ (r & 31)) << 4)) = v;
          }
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float lo = __uint_as_float(u[g * 8 + 2 * q]) * inv_sc;
              const float hi = __uint_as_float(u[g * 8 + 2 * q + 1]) * inv_sc;
              if constexpr (kBF16) {
                __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi);
                w[q] = *reinterpret_cast<uint32_t*>(&t2);
              } else {
                __half2 t2 = __floats2half2_rn(lo, hi);
                w[q] = *reinterpret_cast<uint32_t*>(&t2);
              }
            }
            const int chunk = c * 4 + g;
            *reinterpret_cast<uint4*>(stage + (chunk >> 3) * kHalfBytes + sw128_offset(r, chunk & 7)) =
                make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars.acc_empty[buf]));
      if constexpr (kOutF32) {
        named_bar_sync(1, 128);
        // coalesced copy-out: every warp writes whole 512-byte rows
        for (int rr = wq; rr < kTile; rr += 4) {
          const int s = s0 + rr;
          if (s < p.S) {
            const float4 v = *reinterpret_cast<const float4*>(stage + rr * 512 + (lane << 4));
            const int chunk = lane ^ (rr & 31);
            float* o = p.out_f32 + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(s) * p.o_ss +
                       static_cast<int64_t>(h) * p.o_sh + chunk * 4;
            *reinterpret_cast<float4*>(o) = v;
          }
        }
      } else {
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&bars.out_ready[i % kQ]));
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// All three steps in one persistent kernel (SimA; the launch picks it when there are enough
// (batch, head) units to keep every group busy).  Four CTAs form a group that walks units; each
// CTA owns a quarter of the sequence of the unit at hand:
//   phase 1  statistics over its slab as in sima_stats_kernel, partial results into the group's
//            slots of the workspace (a few MB for the whole grid: they never leave L2);
//   barrier  a counter per unit, bounded wait;
//   reduce   every CTA sums the four partials in slab order, normalises and writes M'' straight
//            into its own shared memory in the layout the tensor pipe reads (same arithmetic, same
//            order and same per-block scales as sima_reduce_kernel, so the same bits);
//   phase 2  out = (Q M'') * inverse scale over the SAME slab, latest tile first.
// The point is the second read of Q: it comes a few tens of microseconds after the first, from
// the same 0.5 MB slab, while about 37 units are in flight; K and V are loaded with an
// evict-first L2 policy, so Q (2 MB per unit) is still in L2 and the kernel's DRAM traffic is the
// algorithmic minimum: q, k, v once in, out once out.  The grid is at most one CTA per SM, so
// every CTA of a group is resident and the group barrier cannot starve.
// ---------------------------------------------------------------------------------------------
constexpr int kFuThreads = 384;  // warp 0 producer, warp 1 MMA, warps 4-11 statistics and reduce, warps 4-7 epilogue
constexpr int kFuGroup = 4;      // CTAs per unit = blocks of 32 output channels in the reduce
constexpr uint32_t kFuSmem = 7 * kTileBytes + 1024;  // phase 1: 2 x [K|V|Q]; phase 2: M'', 4 Q stages, 2 staging
static_assert(kFuGroup == 4, "the reduce below assigns one block of 32 output channels per partial slot");

struct FusedParams {
  int B, H, S;
  int n_units, n_groups;
  int ntiles, tiles_per_cta;
  float* part_m;      // [n_groups][4][e][d]
  float* part_c;      // [n_groups][4][2][128]
  uint32_t* arrive;   // [n_units], zero at launch: CTAs of the unit whose partials are written
  uint32_t* rdone;    // [n_units], zero at launch: CTAs of the unit that have read all partials
  float* out_f32;
  int64_t o_sb, o_ss, o_sh;
  uint32_t* status;
  uint32_t stagger_ns;  // head start of the even groups over the odd ones
};

struct FuBars {
  uint64_t full[4], empty[4], m_done;  // (four phase-1 stages)
  uint64_t q_full[4], q_empty[4], acc_full[2], acc_empty[2];
};

// waits (bounded) until *ctr >= want; false on time-out
__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t want, volatile uint32_t* abort_flag) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu(ctr) < want) {
    if (((++spins) & 31u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > SM100_WAIT_NS) {
        *abort_flag = 1u;
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}

template <bool kBF16, bool kOutF32>
__global__ void __launch_bounds__(kFuThreads, 1)
sima_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q64,
                  const __grid_constant__ CUtensorMap map_k64, const __grid_constant__ CUtensorMap map_v64,
                  const __grid_constant__ CUtensorMap map_o, const FusedParams p) {
  // Phase 1 streams 64 rows of [K | V | Q] per stage through four stages: the consumers are fast, so
  // about three stages (144 KB) are in flight per SM, which is what the HBM latency asks for;
  // two stages of 128 rows leave one in flight and the kernel latency-bound at 0.8 of the bandwidth.
  constexpr int kSt = 4, kQ = 4;
  constexpr int kRows1 = 64;
  constexpr uint32_t kSubBytes = kRows1 * 128 * 2;  // one operand's 64 rows: two 64-column halves
  constexpr uint32_t kSubHalf = kSubBytes / 2;
  constexpr uint32_t kStageBytes = 3 * kSubBytes;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) FuBars bars;
  __shared__ float inv_c[kTile];
  __shared__ float wmax[4][8];
  __shared__ float inv4_s[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sM = smem_base;                  // phase 2 layout
  const uint32_t sQ = smem_base + kTileBytes;
  const uint32_t sO = sQ + kQ * kTileBytes;
  // phase 1's cross-warp sums sit behind its two stages, in memory phase 2 uses for staging
  float (*red)[8][kTile] = reinterpret_cast<float (*)[8][kTile]>(smem_gen + kSt * kStageBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;
  const int group = static_cast<int>(blockIdx.x) / kFuGroup;
  const int c = static_cast<int>(blockIdx.x) % kFuGroup;
  const int tile0 = c * p.tiles_per_cta;
  const int ntile = max(0, min(p.tiles_per_cta, p.ntiles - tile0));
  float* my_pm = p.part_m + (static_cast<size_t>(group) * kFuGroup + c) * kMElems;
  float* my_pc = p.part_c + (static_cast<size_t>(group) * kFuGroup + c) * 2 * kTile;
  const float* grp_pm = p.part_m + static_cast<size_t>(group) * kFuGroup * kMElems;
  const float* grp_pc = p.part_c + static_cast<size_t>(group) * kFuGroup * 2 * kTile;

  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < kSt; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), 1 + 8);
    }
    mbar_init(smem_u32(&bars.m_done), 1);
    for (int i = 0; i < kQ; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.acc_full[i]), 1);
      mbar_init(smem_u32(&bars.acc_empty[i]), 256);
    }
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_q64);
    tma_prefetch_desc(&map_k64);
    tma_prefetch_desc(&map_v64);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_s), 512);  // M accumulator | two output accumulators
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tM = tmem_base_s, tAcc = tmem_base_s + 128;
  // Every group does the same work per unit, so all of them would switch between the read-heavy
  // first phase and the write-heavy second one at the same moments, and the memory system would
  // idle through every switch and every group barrier.  Odd groups therefore start a little under
  // half a unit late, once; after that the two halves of the grid stay out of step and fill each
  // other's gaps (measured at B8 H32 S8192: 455 -> 421 us).
  if (group & 1) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < p.stagger_ns) __nanosleep(500);
  }
  const uint64_t evict_first = l2_policy_evict_first();
  const uint64_t evict_last = l2_policy_evict_last();

  // Counts that run on over the units, from which ring stages and barrier parities follow; every
  // role advances them the same way (ntile is the same for every unit of this CTA).
  uint32_t n1 = 0, n2 = 0, nu = 0;  // phase-1 steps, phase-2 tiles, units done so far
  int prev_u = -1;
  int pre2 = 0;  // (producer thread) phase-2 tiles already requested during phase 1's tail
  bool ok = true;
  const int nstep = ntile * (kTile / kRows1);  // phase-1 steps of 64 rows

  for (int u = group; u < p.n_units; u += p.n_groups, n1 += nstep, n2 += ntile, ++nu) {
    const int b = u / p.H, h = u % p.H;
    // ------------------------------------------------------------------------------ phase 1
    if (warp == 0) {
      if (lane == 0) {
        for (int i = 0; i < nstep; ++i) {
          const uint32_t k = n1 + i;
          const int st = k % kSt;
          if (k >= kSt && !mbar_wait(smem_u32(&bars.empty[st]), (k / kSt - 1) & 1, abortp)) {
            record_timeout(p.status, 61);
            break;
          }
          const uint32_t bar = smem_u32(&bars.full[st]);
          const uint32_t base = smem_base + st * kStageBytes;
          const int s0 = tile0 * kTile + i * kRows1;
          mbar_expect_tx(bar, kStageBytes);
          tma_load_4d_hint(base, &map_k64, bar, 0, h, s0, b, evict_first);
          tma_load_4d_hint(base + kSubHalf, &map_k64, bar, 64, h, s0, b, evict_first);
          tma_load_4d_hint(base + kSubBytes, &map_v64, bar, 0, h, s0, b, evict_first);
          tma_load_4d_hint(base + kSubBytes + kSubHalf, &map_v64, bar, 64, h, s0, b, evict_first);
          tma_load_4d_hint(base + 2 * kSubBytes, &map_q64, bar, 0, h, s0, b, evict_last);
          tma_load_4d_hint(base + 2 * kSubBytes + kSubHalf, &map_q64, bar, 64, h, s0, b, evict_last);
        }
        // Once every stage of this unit has been consumed (by the MMA and by the column sums) the
        // first Q tiles of phase 2 are requested at once, so that they arrive while the group
        // barrier and the reduce run; the rest follow in phase 2 proper.
        bool drained = true;
        for (int i = max(0, nstep - kSt); i < nstep && drained; ++i) {
          const uint32_t k = n1 + i;
          drained = mbar_wait(smem_u32(&bars.empty[k % kSt]), (k / kSt) & 1, abortp);
        }
        pre2 = 0;
        if (drained) {
          for (int i = 0; i < ntile && i < kQ; ++i, ++pre2) {
            const uint32_t k = n2 + i;
            const int st = k % kQ;
            if (k >= kQ && !mbar_wait(smem_u32(&bars.q_empty[st]), (k / kQ - 1) & 1, abortp)) break;
            const uint32_t bar = smem_u32(&bars.q_full[st]);
            const int s0 = (tile0 + ntile - 1 - i) * kTile;
            mbar_expect_tx(bar, kTileBytes);
            tma_load_4d_hint(sQ + st * kTileBytes, &map_q, bar, 0, h, s0, b, evict_first);
            tma_load_4d_hint(sQ + st * kTileBytes + kHalfBytes, &map_q, bar, 64, h, s0, b, evict_first);
          }
        } else {
          record_timeout(p.status, 60);
        }
      }
    } else if (warp == 1) {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_MN_MAJOR, UMMA_MN_MAJOR, 128, 128);
      bool good = true;
      for (int i = 0; i < nstep && good; ++i) {
        const uint32_t k = n1 + i;
        const int st = k % kSt;
        good = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[st]), (k / kSt) & 1, abortp));
        if (!good) { if (lane == 0) record_timeout(p.status, 62); break; }
        tc_fence_after_sync();
        const uint32_t base = smem_base + st * kStageBytes;
        const uint64_t adesc = umma_smem_desc_sw128(base, kSubHalf, 1024);              // K
        const uint64_t bdesc = umma_smem_desc_sw128(base + kSubBytes, kSubHalf, 1024);  // V
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < kRows1 / 16; ++kk) {
            const uint64_t off = static_cast<uint64_t>(kk * (2048 >> 4));
            umma_ss(tM, adesc + off, bdesc + off, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars.empty[st]));
        }
        __syncwarp();
      }
      if (good && ntile > 0 && elect_one()) umma_commit(smem_u32(&bars.m_done));
      __syncwarp();
    } else if (warp >= 4) {
      const int which = (warp - 4) >> 2;  // 0 = K, 1 = Q
      const int t128 = tid - 128 - which * 128;
      const int chunk16 = t128 & 15;
      const int rg = t128 >> 4;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      bool good = true;
      for (int i = 0; i < nstep; ++i) {
        const uint32_t k = n1 + i;
        const int st = k % kSt;
        good = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[st]), (k / kSt) & 1, abortp));
        if (!good) { if (lane == 0) record_timeout(p.status, 63); break; }
        const uint8_t* tile = smem_gen + st * kStageBytes + (which ? 2 * kSubBytes : 0) +
                              (chunk16 >> 3) * kSubHalf;
#pragma unroll
        for (int r = 0; r < kRows1 / 8; ++r) {
          const int row = rg + 8 * r;
          const uint4 v = *reinterpret_cast<const uint4*>(tile + sw128_offset(row, chunk16 & 7));
          abs_acc8<kBF16>(v, acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.empty[st]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) red[which][rg][chunk16 * 8 + i] = acc[i];
      named_bar_sync(1 + which, 128);
      // the group's slots still hold the previous unit's partials until every CTA of the group has
      // read them (by now it has, long ago; the wait costs one load)
      if (prev_u >= 0 && good) good = wait_counter(p.rdone + prev_u, kFuGroup, abortp);
      float sum = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) sum += red[which][g][t128];
      my_pc[which * kTile + t128] = sum;
      if (which == 0) {
        const int wq = warp & 3;
        const int d = wq * 32 + lane;
        if (ntile > 0) {
          good = good && __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.m_done), nu & 1, abortp));
          if (good) {
            tc_fence_after_sync();
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t uu[32];
              tmem_ld32(tM + (static_cast<uint32_t>(wq * 32) << 16) + cc * 32, uu);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) my_pm[(cc * 32 + i) * kTile + d] = __uint_as_float(uu[i]);
            }
          } else if (lane == 0) {
            record_timeout(p.status, 64);
          }
        } else {
          for (int i = 0; i < 128; ++i) my_pm[i * kTile + d] = 0.f;
        }
      }
      if (!good) *abortp = 1u;
    }
    // ------------------------------------------------------------------------------ group barrier
    __threadfence();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0) {
      atomicAdd(p.arrive + u, 1u);
      if (!wait_counter(p.arrive + u, kFuGroup, abortp)) record_timeout(p.status, 65);
    }
    __syncthreads();
    if (*abortp) { ok = false; break; }
    // ------------------------------------------------------------------------------ reduce
    if (warp >= 4) {
      const int t256 = tid - 128;
      if (t256 < kTile) {
        float ck = 0.f, cq = 0.f;
        for (int cc = 0; cc < kFuGroup; ++cc) {
          ck += __ldcg(grp_pc + (cc * 2 + 0) * kTile + t256);
          cq += __ldcg(grp_pc + (cc * 2 + 1) * kTile + t256);
        }
        inv_c[t256] = __fdiv_rn(1.0f, __fmul_rn(ck, cq));
      }
      named_bar_sync(3, 256);
      float vals[4][16];
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        float amax = 0.f;
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int idx = it * 256 + t256;  // = e_local * 128 + d
          float m = 0.f;
#pragma unroll
          for (int cc = 0; cc < kFuGroup; ++cc) m += __ldcg(grp_pm + static_cast<size_t>(cc) * kMElems + blk * kRedElems + idx);
          m *= inv_c[idx & 127];
          vals[blk][it] = m;
          amax = fmaxf(amax, fabsf(m));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0) wmax[blk][warp - 4] = amax;
      }
      __threadfence();
      named_bar_sync(3, 256);
      if (t256 == 0) atomicAdd(p.rdone + u, 1u);  // every partial of this unit has been read by this CTA
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a = fmaxf(a, wmax[blk][i]);
        float sc = 1.f;
        if (a > 0.f && a < INFINITY) {
          int ex;
          frexpf(a, &ex);
          sc = ldexpf(1.0f, 14 - ex);
        }
        if (t256 == 0) inv4_s[blk] = 1.0f / sc;
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int idx = it * 256 + t256;
          const int e = blk * 32 + (idx >> 7), d = idx & 127;
          const float v = vals[blk][it] * sc;
          uint16_t bits;
          if constexpr (kBF16) {
            __nv_bfloat16 hb = __float2bfloat16_rn(v);
            bits = *reinterpret_cast<uint16_t*>(&hb);
          } else {
            __half hh = __float2half_rn(v);
            bits = *reinterpret_cast<uint16_t*>(&hh);
          }
          // M''^T [e][d], d contiguous: the K-major B operand, two 64-element halves, 128-byte swizzle
          *reinterpret_cast<uint16_t*>(smem_gen + (d >> 6) * kHalfBytes + sw128_offset(e, (d & 63) >> 3) + (d & 7) * 2) = bits;
        }
      }
      fence_proxy_async_smem();  // written by ordinary stores, read by the tensor pipe
    }
    __syncthreads();
    // ------------------------------------------------------------------------------ phase 2
    if (warp == 0) {
      if (lane == 0) {
        for (int i = pre2; i < ntile; ++i) {
          const uint32_t k = n2 + i;
          const int st = k % kQ;
          if (k >= kQ && !mbar_wait(smem_u32(&bars.q_empty[st]), (k / kQ - 1) & 1, abortp)) {
            record_timeout(p.status, 66);
            break;
          }
          const uint32_t bar = smem_u32(&bars.q_full[st]);
          const int s0 = (tile0 + ntile - 1 - i) * kTile;  // latest tile first: the freshest in L2
          mbar_expect_tx(bar, kTileBytes);
          tma_load_4d_hint(sQ + st * kTileBytes, &map_q, bar, 0, h, s0, b, evict_first);
          tma_load_4d_hint(sQ + st * kTileBytes + kHalfBytes, &map_q, bar, 64, h, s0, b, evict_first);
        }
      }
    } else if (warp == 1) {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
      const uint64_t mdesc = umma_smem_desc_sw128(sM, 16, 1024);
      bool good = true;
      for (int i = 0; i < ntile && good; ++i) {
        const uint32_t k = n2 + i;
        const int st = k % kQ, buf = k & 1;
        good = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.q_full[st]), (k / kQ) & 1, abortp));
        if (good && k >= 2)
          good = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_empty[buf]), ((k >> 1) - 1) & 1, abortp));
        if (!good) { if (lane == 0) record_timeout(p.status, 67); break; }
        tc_fence_after_sync();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ + st * kTileBytes, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
            umma_ss(tAcc + buf * 128, qdesc + off, mdesc + off, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars.acc_full[buf]));
          umma_commit(smem_u32(&bars.q_empty[st]));
        }
        __syncwarp();
      }
    } else if (warp >= 4) {
      // Eight epilogue warps: two per TMEM lane quarter, each with half of the 128 output columns
      // (four warps alone finish a tile in about 1.5 us, which held this phase to half of the
      // SM's share of the memory bandwidth).
      const int wq = warp & 3;
      const int ch0 = ((warp - 4) >> 2) * 2;  // this warp's two chunks of 32 columns: 0,1 or 2,3
      const int r = wq * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
      const float inv4[4] = {inv4_s[0], inv4_s[1], inv4_s[2], inv4_s[3]};
      bool good = true;
      for (int i = 0; i < ntile && good; ++i) {
        const uint32_t k = n2 + i;
        const int buf = k & 1;
        const int s0 = (tile0 + ntile - 1 - i) * kTile;
        good = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_full[buf]), (k >> 1) & 1, abortp));
        if (!good) { if (lane == 0) record_timeout(p.status, 68); break; }
        tc_fence_after_sync();
        if constexpr (!kOutF32) {
          if (tid == 128) tma_store_wait_read_n<1>();
        }
        named_bar_sync(1, 256);
        uint8_t* stage = smem_gen + (sO - smem_base) + (kOutF32 ? 0 : buf * kTileBytes);
#pragma unroll
        for (int cc = ch0; cc < ch0 + 2; ++cc) {
          uint32_t uu[32];
          tmem_ld32(tAcc + lane_base + buf * 128 + cc * 32, uu);
          tmem_wait_ld();
          const float inv_sc = inv4[cc];
          if constexpr (kOutF32) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              float4 v;
              v.x = __uint_as_float(uu[g * 4 + 0]) * inv_sc;
              v.y = __uint_as_float(uu[g * 4 + 1]) * inv_sc;
              v.z = __uint_as_float(uu[g * 4 + 2]) * inv_sc;
              v.w = __uint_as_float(uu[g * 4 + 3]) * inv_sc;
              const int chunk = cc * 8 + g;
              *reinterpret_cast<float4*>(stage + r * 512 + ((chunk ^ (r & 31)) << 4)) = v;
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float lo = __uint_as_float(uu[g * 8 + 2 * q]) * inv_sc;
                const float hi = __uint_as_float(uu[g * 8 + 2 * q + 1]) * inv_sc;
                if constexpr (kBF16) {
                  __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi);
                  w[q] = *reinterpret_cast<uint32_t*>(&t2);
                } else {
                  __half2 t2 = __floats2half2_rn(lo, hi);
                  w[q] = *reinterpret_cast<uint32_t*>(&t2);
                }
              }
              const int chunk = cc * 4 + g;
              *reinterpret_cast<uint4*>(stage + (chunk >> 3) * kHalfBytes + sw128_offset(r, chunk & 7)) =
                  make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bars.acc_empty[buf]));
        if constexpr (kOutF32) {
          named_bar_sync(1, 256);
          for (int rr = warp - 4; rr < kTile; rr += 8) {
            const int srow = s0 + rr;
            if (srow < p.S) {
              const float4 v = *reinterpret_cast<const float4*>(stage + rr * 512 + (lane << 4));
              const int chunk = lane ^ (rr & 31);
              float* o = p.out_f32 + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(srow) * p.o_ss +
                         static_cast<int64_t>(h) * p.o_sh + chunk * 4;
              *reinterpret_cast<float4*>(o) = v;
            }
          }
        } else {
          fence_proxy_async_smem();
          named_bar_sync(1, 256);
          if (tid == 128) {
#ifdef ASUKA_SIMA_STORE_PLAIN
            tma_store_4d(&map_o, sO + buf * kTileBytes, 0, h, s0, b);
            tma_store_4d(&map_o, sO + buf * kTileBytes + kHalfBytes, 64, h, s0, b);
#else
            tma_store_4d_hint(&map_o, sO + buf * kTileBytes, 0, h, s0, b, evict_first);
            tma_store_4d_hint(&map_o, sO + buf * kTileBytes + kHalfBytes, 64, h, s0, b, evict_first);
#endif
            tma_store_commit();
          }
        }
      }
      if constexpr (!kOutF32) {
        if (tid == 128) tma_store_wait_read();  // phase 1 of the next unit reuses the staging memory
      }
      if (!good) *abortp = 1u;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (*abortp) { ok = false; break; }
    prev_u = u;
  }
  (void)ok;
  (void)evict_last;

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base_s, 512);
  }
}

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct Plan {
  int ntiles, nchunks, tiles_per_chunk;
  size_t off_pm, off_pc, off_m16, off_sc, off_cnt, total;
};

// Into how many slabs the sequence of one (batch, head) unit is cut for the statistics and for the
// output kernel of the three-kernel path: about seven waves of CTAs on a 148-SM part, but at least
// eight tiles per CTA -- filling and draining the stage ring and loading M'' cost a CTA about as
// much as four tiles -- unless that would leave SMs without a CTA.
int slabs_per_unit(int bh, int ntiles) {
  int want = (1024 + bh - 1) / bh;
  const int long_enough = ntiles / 8 > 1 ? ntiles / 8 : 1;
  if (want > long_enough) want = long_enough;
  const int fill = (148 + bh - 1) / bh;
  if (want < fill) want = fill;
  if (want > ntiles) want = ntiles;
  return want < 1 ? 1 : want;
}

Plan make_plan(const SimaShape& s) {
  Plan pl;
  const int bh = s.B * s.H;
  pl.ntiles = (s.S + kTile - 1) / kTile;
  int want = slabs_per_unit(bh, pl.ntiles);
  if (want > kMaxChunks) want = kMaxChunks;
  pl.tiles_per_chunk = (pl.ntiles + want - 1) / want;
  pl.nchunks = (pl.ntiles + pl.tiles_per_chunk - 1) / pl.tiles_per_chunk;
  size_t off = 0;
  pl.off_pm = off; off = align256(off + static_cast<size_t>(bh) * pl.nchunks * kMElems * 4);
  pl.off_pc = off; off = align256(off + static_cast<size_t>(bh) * pl.nchunks * 2 * kTile * 4);
  pl.off_m16 = off; off = align256(off + static_cast<size_t>(bh) * kMElems * 2);
  pl.off_sc = off; off = align256(off + static_cast<size_t>(bh) * kRedBlocks * 4);
  pl.off_cnt = off; off = align256(off + static_cast<size_t>(bh) * 2 * sizeof(uint32_t));  // fused kernel's counters
  pl.total = off;
  return pl;
}

}  // namespace

size_t sima_workspace_bytes(const SimaShape& s) { return make_plan(s).total; }


cudaError_t launch_sima(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mo, void* out_ptr, int64_t out_stride_b,
                        int64_t out_stride_s, int64_t out_stride_h, void* ws, const SimaShape& s,
                        const CUtensorMap* maps64, int num_sms, cudaStream_t stream) {
  const Plan pl = make_plan(s);
  const int bh = s.B * s.H;
  uint8_t* w = static_cast<uint8_t*>(ws);
  // One persistent kernel for all three steps when there are enough units to keep most groups of
  // four CTAs busy (and the partial slots fit the workspace plan above).
  const int n_groups = num_sms / kFuGroup;
#ifdef ASUKA_SIMA_NO_FUSED
  const bool fused = false;
#else
  const bool fused = !s.ea && maps64 != nullptr && n_groups > 0 && 2 * bh >= n_groups && pl.ntiles >= kFuGroup &&
                     static_cast<long long>(bh) * pl.nchunks >= static_cast<long long>(n_groups) * kFuGroup;
#endif
  if (fused) {
    FusedParams fp;
    fp.B = s.B; fp.H = s.H; fp.S = s.S;
    fp.n_units = bh;
    fp.n_groups = n_groups;
    fp.ntiles = pl.ntiles;
    fp.tiles_per_cta = (pl.ntiles + kFuGroup - 1) / kFuGroup;
    fp.part_m = reinterpret_cast<float*>(w + pl.off_pm);
    fp.part_c = reinterpret_cast<float*>(w + pl.off_pc);
    fp.arrive = reinterpret_cast<uint32_t*>(w + pl.off_cnt);
    fp.rdone = fp.arrive + bh;
    fp.out_f32 = s.out_f32 ? static_cast<float*>(out_ptr) : nullptr;
    fp.o_sb = out_stride_b; fp.o_ss = out_stride_s; fp.o_sh = out_stride_h;
    fp.status = device_status_words();
    {
      // a unit costs a CTA five passes over its slab (K, V, Q in; Q again from L2; out) at its
      // share of the memory bandwidth, about 44 bytes per nanosecond per SM on this part
      const double unit_ns = static_cast<double>(fp.tiles_per_cta) * kTile * 128 * 2 * 5 / 44.0;
      // (with fewer than three rounds of units the head start costs more than it brings)
      fp.stagger_ns = bh >= 3 * n_groups ? static_cast<uint32_t>(0.4 * unit_ns) : 0u;
    }
    cudaError_t e = cudaMemsetAsync(fp.arrive, 0, static_cast<size_t>(bh) * 2 * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, FusedParams);
    if (s.out_f32) kern = s.bf16 ? sima_fused_kernel<true, true> : sima_fused_kernel<false, true>;
    else kern = s.bf16 ? sima_fused_kernel<true, false> : sima_fused_kernel<false, false>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(kFuSmem));
    if (e != cudaSuccess) return e;
    kern<<<static_cast<unsigned>(n_groups * kFuGroup), kFuThreads, kFuSmem, stream>>>(mq, maps64[0], maps64[1], maps64[2],
                                                                                      s.out_f32 ? mq : mo, fp);
    count_launch();
    return cudaGetLastError();
  }
  StatsParams sp;
  sp.B = s.B; sp.H = s.H; sp.S = s.S;
  sp.nchunks = pl.nchunks; sp.tiles_per_chunk = pl.tiles_per_chunk; sp.ntiles = pl.ntiles;
  sp.ws.part_m = reinterpret_cast<float*>(w + pl.off_pm);
  sp.ws.part_c = reinterpret_cast<float*>(w + pl.off_pc);
  sp.ws.m16 = reinterpret_cast<uint16_t*>(w + pl.off_m16);
  sp.ws.inv_scale = reinterpret_cast<float*>(w + pl.off_sc);
  sp.ea = s.ea ? 1 : 0;
  sp.status = device_status_words();

  cudaError_t e;
  {
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, StatsParams);
    if (s.ea) kern = s.bf16 ? sima_stats_kernel<true, true> : sima_stats_kernel<false, true>;
    else kern = s.bf16 ? sima_stats_kernel<true, false> : sima_stats_kernel<false, false>;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kStSmem);
    if (e != cudaSuccess) return e;
    kern<<<static_cast<unsigned>(bh) * pl.nchunks, kStThreads, kStSmem, stream>>>(mq, mk, mv, sp);
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  {
    auto kern = s.bf16 ? sima_reduce_kernel<true> : sima_reduce_kernel<false>;
    kern<<<bh * kRedBlocks, 256, 0, stream>>>(sp);
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  {
    CUtensorMap mm;
    if (tma_host::make_bshd_map(&mm, sp.ws.m16, s.bf16, 1, static_cast<int64_t>(bh) * kTile, 1, kTile,
                                static_cast<int64_t>(bh) * kMElems, kTile, kTile, 128) != 0)
      return cudaErrorInvalidValue;
    OutParams op;
    op.B = s.B; op.H = s.H; op.S = s.S;
    op.ntiles = pl.ntiles;
    const int nq = slabs_per_unit(bh, pl.ntiles);
    op.tiles_per_cta = (pl.ntiles + nq - 1) / nq;
    op.nqchunks = (pl.ntiles + op.tiles_per_cta - 1) / op.tiles_per_cta;
    op.inv_scale = sp.ws.inv_scale;
    op.out_f32 = s.out_f32 ? static_cast<float*>(out_ptr) : nullptr;
    op.o_sb = out_stride_b; op.o_ss = out_stride_s; op.o_sh = out_stride_h;
    op.status = sp.status;
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, OutParams);
    if (s.ea) {
      if (s.out_f32) kern = s.bf16 ? sima_out_kernel<true, true, true> : sima_out_kernel<false, true, true>;
      else kern = s.bf16 ? sima_out_kernel<true, false, true> : sima_out_kernel<false, false, true>;
    } else {
      if (s.out_f32) kern = s.bf16 ? sima_out_kernel<true, true, false> : sima_out_kernel<false, true, false>;
      else kern = s.bf16 ? sima_out_kernel<true, false, false> : sima_out_kernel<false, false, false>;
    }
    const uint32_t out_smem = out_smem_bytes(s.out_f32, s.ea);
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(out_smem));
    if (e != cudaSuccess) return e;
    kern<<<static_cast<unsigned>(bh) * op.nqchunks, kOutThreads + (s.ea ? 256 : 0), out_smem, stream>>>(mq, mm, s.out_f32 ? mq : mo, op);
    count_launch();
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace asuka
