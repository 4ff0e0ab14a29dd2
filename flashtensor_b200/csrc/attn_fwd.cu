// Attention forward for sm_100a: O = softmax(Q K^T * scale + causal mask) V, plus the per-row
// base-2 log-sum-exp that the column-score pass consumes.
//
// Replaces the kernel the Asuka pipeline generates for Attn.forward (cases/kernels/attn.py:18-34):
// f32 exp2-based softmax with the division deferred until after P.V, P rounded to the input type
// for the second product, f32 accumulation, fully masked tiles skipped (the numerics fixed by
// LowerComplexReduce / RecoverTypeInKernel / ReplaceExpAndLog / EquivalentTransform / DynamicFor).
//
// The kernel is persistent: one CTA per SM walks a list of work items (256 query rows of one
// (batch, head), heaviest first, dealt out in a zigzag so that every CTA gets the same amount of
// work).  The two 128-row tiles of an item ping-pong through the tensor pipe so that the softmax of
// one overlaps the MMAs of the other, and the K/V/Q loads and the first QK^T of the next item run
// under the tail and the epilogue of the current one.
//   warp 0        TMA producer: Q once, then K tiles of 128 keys through a 3-stage ring
//   warp 2        TMA producer: V tiles through a 2-stage ring
//   warp 1        issues tcgen05.mma: S_t = Q_t K^T (SMEM x SMEM), O_t += P_t V (TMEM x SMEM)
//   warps 4-7     softmax of tile 0: one thread per query row, whole row of S in registers
//   warps 8-11    softmax of tile 1
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 f32 columns each; P_t (16-bit, 64 columns)
// overwrites the front of S_t once S_t is in registers.  The exponent reference of a row is only
// taken from the first tile's true row maximum and then only moved when a later tile's row sum
// would overflow the stale one, so O is rescaled (a TMEM round trip) almost never.  The epilogue writes O_t / l from registers straight to global memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "kernels.h"
#include "sm100_ptx.cuh"

namespace asuka {
using namespace sm100;

namespace {

constexpr int kTile = 128;
constexpr uint32_t kTileBytes = 128 * 128 * 2;  // one [128 x 128] 16-bit tile = two swizzled halves
constexpr uint32_t kHalfBytes = kTileBytes / 2;
constexpr int kKStages = 3;  // K(j) is needed one iteration before V(j): give it the deeper ring
constexpr int kVStages = 2;
constexpr int kThreads = 384;
constexpr int kUtilRegs = 96;      // 128 * 96 + 256 * 200 = 63488 <= 384 * 168
constexpr int kSoftmaxRegs = 200;
constexpr uint32_t kSmemBytes = (2 + kKStages + kVStages) * kTileBytes + 1024;
constexpr float kRescaleLimit = 8192.0f;  // largest tile row sum tolerated under a stale reference:
                                          // bounds every exponential far below fp16's 65504

struct FwdParams {
  int B, H, Sq, Skv;
  int causal, diag_off;
  int nq_blocks, n_items;
  int pair_far, nq_tiles;    // pair_far: an item is the query tiles i and nq_tiles - 1 - i (see decode_item)
  int unit_major;            // items are numbered unit by unit instead of heaviest block first
  int group;                 // query heads per key/value head (grouped-query attention)
  float scale_log2;          // softmax_scale * log2(e)
  float cap_in, cap_out;     // soft-capping: softmax_scale / cap and cap * log2(e)
  float* lse2;
  void* out;                 // [B, Sq, H, 128], 16-bit, strides in elements
  int64_t o_sb, o_ss, o_sh;
  int out_vec32;             // every output row starts on a 32-byte boundary: 256-bit stores
  uint32_t* status;
  // Key-range split, for launches with fewer work items than SMs can share evenly: the keys of
  // every item are dealt out to `parts` items of `ceil(n / parts)` key tiles each.  A query tile
  // served by more than one part leaves, per part, its unnormalised O (f32), its exponent
  // reference and its row sum in the workspace; attn_merge_kernel combines them in part order.
  int parts;
  float* part_o;             // [B*H, Sq, parts, 128]
  float* part_ml;            // [B*H, Sq, parts, 2]
};

struct Bars {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[kKStages], k_empty[kKStages];
  uint64_t v_full[kVStages], v_empty[kVStages];
  uint64_t s_full[2], p_ready[2], o_done[2], o_free[2];
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 256-bit store: one instruction per 32-byte sector instead of two (the epilogue's stores go to 32
// different rows per warp instruction, so the number of instructions is what the LSU pays for)
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool kBF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool kBF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (kBF16) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
}

__device__ __forceinline__ void record_timeout(uint32_t* status, uint32_t site) {
  atomicAdd(&status[0], 1u);
  status[1] = site;
}

// number of 128-key tiles query tile [q0, q0+128) has to visit
__host__ __device__ __forceinline__ int kv_tiles_for(int q0, const FwdParams& p) {
  if (q0 >= p.Sq) return 0;
  int last = p.Skv - 1;
  if (p.causal) {
    const int qlast = q0 + kTile - 1 < p.Sq - 1 ? q0 + kTile - 1 : p.Sq - 1;
    last = last < qlast + p.diag_off ? last : qlast + p.diag_off;
  }
  return last / kTile + 1;
}


// One work item: 256 query rows of one (batch, head).
struct Item {
  int b, h;
  int q0[2];      // first row of each 128-row tile
  int j0;         // first key tile of this item (0 unless the keys are split)
  int n_kv[2];    // 128-key tiles each tile visits from j0 on (0: nothing for this tile in this item)
  int n_max;
  int part;       // which part of the key range this item is
  int nparts[2];  // parts that serve each tile (1: this item writes the tile's final result)
};

// Item `idx` of the launch; items are numbered heaviest first.  kSplit = false is the common case
// of one item per 256-row block, compiled without any of the key-range arithmetic (which costs
// the softmax warps registers they do not have).
template <bool kSplit>
__device__ __forceinline__ void decode_item(int idx, const FwdParams& p, Item* item) {
  const int bh_count = p.B * p.H;
  if constexpr (!kSplit) {
    // unit_major: the blocks of one (batch, head) follow each other, latest first, so that they
    // run at about the same time and K/V are in L2 for all but the first of them.  It is used
    // when K and V of the whole launch do not fit L2 (otherwise every wave of blocks would fetch
    // them from DRAM again).
    const int bh = p.unit_major ? idx / p.nq_blocks : idx % bh_count;
    item->b = bh / p.H;
    item->h = bh % p.H;
    if (p.unit_major) {
      const int qb = p.nq_blocks - 1 - idx % p.nq_blocks;
      item->q0[0] = qb * 2 * kTile;
      item->q0[1] = qb * 2 * kTile + kTile;
    } else if (p.pair_far) {
      // A causal launch that fills at most one wave ends with its heaviest item, and items of
      // adjacent tiles grow with the block index.  Pairing tile i with tile nq_tiles - 1 - i makes
      // every item nq_tiles + 1 tile steps: the early tile shares the first key tiles with the
      // late one, which then runs on alone.
      const int i = idx / bh_count, far = p.nq_tiles - 1 - i;
      item->q0[0] = i * kTile;
      item->q0[1] = far > i ? far * kTile : p.Sq;  // (an odd count leaves the middle tile alone)
    } else {
      const int qb = p.nq_blocks - 1 - idx / bh_count;
      item->q0[0] = qb * 2 * kTile;
      item->q0[1] = qb * 2 * kTile + kTile;
    }
    item->j0 = 0;
    item->n_kv[0] = kv_tiles_for(item->q0[0], p);
    item->n_kv[1] = kv_tiles_for(item->q0[1], p);
    item->n_max = max(item->n_kv[0], item->n_kv[1]);
    item->part = 0;
    item->nparts[0] = item->nparts[1] = 1;
    return;
  }
  const int per_block = bh_count * p.parts;
  const int qb = p.nq_blocks - 1 - idx / per_block;
  const int rem = idx % per_block;
  const int bh = rem % bh_count;
  item->part = rem / bh_count;
  item->b = bh / p.H;
  item->h = bh % p.H;
  item->q0[0] = qb * 2 * kTile;
  item->q0[1] = qb * 2 * kTile + kTile;
  const int full0 = kv_tiles_for(item->q0[0], p), full1 = kv_tiles_for(item->q0[1], p);
  const int full = full0 > full1 ? full0 : full1;
  const int len = (full + p.parts - 1) / p.parts;  // key tiles per part (>= 1)
  item->j0 = item->part * len;
  const int r0 = full0 - item->j0 < len ? full0 - item->j0 : len;
  const int r1 = full1 - item->j0 < len ? full1 - item->j0 : len;
  item->n_kv[0] = r0 > 0 ? r0 : 0;
  item->n_kv[1] = r1 > 0 ? r1 : 0;
  item->n_max = item->n_kv[0] > item->n_kv[1] ? item->n_kv[0] : item->n_kv[1];
  item->nparts[0] = (full0 + len - 1) / len;
  item->nparts[1] = (full1 + len - 1) / len;
}

// The it-th item of this CTA: wave w of gridDim.x items is dealt out forwards when w is even and
// backwards when it is odd, which evens out the totals (at 32 heads and S = 4096 the busiest CTA
// gets 3 % more than the mean; assigning longest-first to the least-loaded CTA on the host would
// get within 2.5 %, the items being as coarse as they are, and was not worth a table).
template <bool kSplit>
__device__ __forceinline__ bool get_item(int it, const FwdParams& p, Item* item) {
  const int G = static_cast<int>(gridDim.x);
  const int r = static_cast<int>(blockIdx.x);
  const int idx = it * G + ((it & 1) ? G - 1 - r : r);
  if (idx >= p.n_items) return false;
  decode_item<kSplit>(idx, p, item);
  return true;
}
// with an odd number of waves the last, backwards-dealt wave can skip a CTA that still has none
__device__ __forceinline__ int item_waves(const FwdParams& p) {
  return (p.n_items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
}

// kCap: Gemma-2 style soft-capping, logits -> cap * tanh(logits / cap) before the mask
// (cases/kernels/gemma2.py:30-33; the reference emits tanh.approx.f32 too, to_triton.cpp:351-369).
template <bool kBF16, bool kCap, bool kSplit>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) Bars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;                          // 2 tiles
  const uint32_t sK = smem_base + 2 * kTileBytes;         // kKStages tiles
  const uint32_t sV = sK + kKStages * kTileBytes;         // kVStages tiles

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile uint32_t* abortp = &abort_s;
  const int n_waves = item_waves(p);

  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 1);
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.p_ready[i]), 128);
      mbar_init(smem_u32(&bars.o_done[i]), 1);
      mbar_init(smem_u32(&bars.o_free[i]), 128);
    }
    for (int i = 0; i < kKStages; ++i) {
      mbar_init(smem_u32(&bars.k_full[i]), 1);
      mbar_init(smem_u32(&bars.k_empty[i]), 1);
    }
    for (int i = 0; i < kVStages; ++i) {
      mbar_init(smem_u32(&bars.v_full[i]), 1);
      mbar_init(smem_u32(&bars.v_empty[i]), 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
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
  // The set-up above may have run while the kernel ahead in the stream was still draining; q, k and
  // v may be that kernel's outputs and out / lse its inputs, so nothing is read or written before
  // it has finished.  The kernel behind this one (the column pass) may be scheduled from now on:
  // its CTAs come up on SMs whose forward CTA has retired and wait there for this grid's end.
  griddep_wait();
  griddep_launch_dependents();

  // Every role walks the same item list and keeps running counts (K tiles, V tiles, tile steps,
  // items per tile) from which ring stages and barrier parities follow; nothing is reset
  // between items.
  // 384 threads x 168 registers: the four utility warps hand most of theirs to the softmax warps
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: Q and K
    reg_dealloc<kUtilRegs>();
    if (lane == 0) {
      bool ok = true;
      uint32_t kc = 0;            // K tiles issued so far
      uint32_t qn[2] = {0, 0};    // items in which tile t was loaded so far
      Item it_;
      for (int it = 0; it < n_waves && ok; ++it) {
        if (!get_item<kSplit>(it, p, &it_)) continue;
        for (int t = 0; t < 2 && ok; ++t) {
          if (it_.n_kv[t] == 0) continue;
          if (qn[t] > 0) {  // the previous item's last QK^T of this tile must have read Q_t
            ok = mbar_wait(smem_u32(&bars.q_empty[t]), (qn[t] - 1) & 1, abortp);
            if (!ok) { record_timeout(p.status, 11); break; }
          }
          const uint32_t bar = smem_u32(&bars.q_full[t]);
          mbar_expect_tx(bar, kTileBytes);
          tma_load_4d(sQ + t * kTileBytes, &map_q, bar, 0, it_.h, it_.q0[t], it_.b);
          tma_load_4d(sQ + t * kTileBytes + kHalfBytes, &map_q, bar, 64, it_.h, it_.q0[t], it_.b);
          ++qn[t];
        }
        for (int j = 0; j < it_.n_max && ok; ++j, ++kc) {
          const int st = kc % kKStages;
          const uint32_t use = kc / kKStages;
          if (use > 0) {
            ok = mbar_wait(smem_u32(&bars.k_empty[st]), (use - 1) & 1, abortp);
            if (!ok) { record_timeout(p.status, 1); break; }
          }
          const uint32_t bar = smem_u32(&bars.k_full[st]);
          mbar_expect_tx(bar, kTileBytes);
          tma_load_4d(sK + st * kTileBytes, &map_k, bar, 0, it_.h / p.group, ((kSplit ? it_.j0 : 0) + j) * kTile, it_.b);
          tma_load_4d(sK + st * kTileBytes + kHalfBytes, &map_k, bar, 64, it_.h / p.group, ((kSplit ? it_.j0 : 0) + j) * kTile, it_.b);
        }
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before the CTA retires
        volatile uint32_t none = 0;
        for (uint32_t c = kc > kKStages ? kc - kKStages : 0; c < kc; ++c)
          mbar_wait(smem_u32(&bars.k_full[c % kKStages]), (c / kKStages) & 1, &none);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ TMA producer: V
    reg_dealloc<kUtilRegs>();
    if (lane == 0) {
      bool ok = true;
      uint32_t vc = 0;
      Item it_;
      for (int it = 0; it < n_waves && ok; ++it) {
        if (!get_item<kSplit>(it, p, &it_)) continue;
        for (int j = 0; j < it_.n_max && ok; ++j, ++vc) {
          const int st = vc % kVStages;
          const uint32_t use = vc / kVStages;
          if (use > 0) {
            ok = mbar_wait(smem_u32(&bars.v_empty[st]), (use - 1) & 1, abortp);
            if (!ok) { record_timeout(p.status, 2); break; }
          }
          const uint32_t bar = smem_u32(&bars.v_full[st]);
          mbar_expect_tx(bar, kTileBytes);
          tma_load_4d(sV + st * kTileBytes, &map_v, bar, 0, it_.h / p.group, ((kSplit ? it_.j0 : 0) + j) * kTile, it_.b);
          tma_load_4d(sV + st * kTileBytes + kHalfBytes, &map_v, bar, 64, it_.h / p.group, ((kSplit ? it_.j0 : 0) + j) * kTile, it_.b);
        }
      }
      if (!ok) {
        volatile uint32_t none = 0;
        for (uint32_t c = vc > kVStages ? vc - kVStages : 0; c < vc; ++c)
          mbar_wait(smem_u32(&bars.v_full[c % kVStages]), (c / kVStages) & 1, &none);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // One warp issues for both tiles, in the order P.V_0(j-1), QK_0(j), P.V_1(j-1), QK_1(j): the
    // S/P aliasing of a tile is ordered by program order, and the two tiles are forced to
    // alternate (their softmax phases share the MUFU, so they must not run in step).  The whole
    // warp walks the loop (addresses and descriptors stay warp-uniform, waits are converged); one
    // elected lane issues the tcgen05.mma / commit instructions.  Barriers that are normally
    // already complete are probed together so that their latencies overlap.
    reg_dealloc<kUtilRegs>();
    {
      constexpr uint32_t kFmt = kBF16 ? UMMA_BF16 : UMMA_F16;
      constexpr uint32_t idesc_qk = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kFmt, UMMA_K_MAJOR, UMMA_MN_MAJOR, 128, 128);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
        const bool good = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, abortp));
        if (!good && lane == 0) record_timeout(p.status, site);
        return good;
      };
      bool ok = true;
      uint32_t kc = 0, vc = 0;      // K / V tiles consumed before this item
      uint32_t sn[2] = {0, 0};      // tile steps of tile t before this item (parity of s_full, p_ready)
      uint32_t on[2] = {0, 0};      // items of tile t before this one (parity of q_full, o_free)
      Item it_;
      for (int it = 0; it < n_waves && ok; ++it) {
        if (!get_item<kSplit>(it, p, &it_)) continue;
        const int n_max = it_.n_max;
        for (int t = 0; t < 2 && ok; ++t) {
          if (it_.n_kv[t] > 0) ok = wait_all(&bars.q_full[t], on[t] & 1, 3);
        }
        for (int j = 0; j <= n_max && ok; ++j) {
          const int jp = j - 1;  // the tile whose P.V is issued in this iteration
          const bool have_k = j < n_max, have_v = jp >= 0;
          const uint32_t kidx = kc + j, vidx = vc + (have_v ? jp : 0);
          const int st = kidx % kKStages, stp = vidx % kVStages;
          const bool pv0 = have_v && jp < it_.n_kv[0], pv1 = have_v && jp < it_.n_kv[1];
          // probe everything this iteration needs at once; fall back to a proper wait on a miss
          const bool k_hit = !have_k || mbar_try_wait(smem_u32(&bars.k_full[st]), (kidx / kKStages) & 1);
          const bool v_hit = !have_v || mbar_try_wait(smem_u32(&bars.v_full[stp]), (vidx / kVStages) & 1);
          const bool p0_hit = !pv0 || mbar_try_wait(smem_u32(&bars.p_ready[0]), (sn[0] + jp) & 1);
          if (!__all_sync(0xffffffffu, k_hit)) ok = wait_all(&bars.k_full[st], (kidx / kKStages) & 1, 4);
          if (ok && !__all_sync(0xffffffffu, v_hit)) ok = wait_all(&bars.v_full[stp], (vidx / kVStages) & 1, 5);
          if (!ok) break;
          const uint64_t kdesc = umma_smem_desc_sw128(sK + st * kTileBytes, 16, 1024);
          const uint64_t vdesc = umma_smem_desc_sw128(sV + stp * kTileBytes, kHalfBytes, 1024);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t tS = tbase + t * 128;          // S_t, and P_t in its first 64 columns
            const uint32_t tO = tbase + 256 + t * 128;    // O_t
            const bool pv = t == 0 ? pv0 : pv1;
            const bool qk = j < it_.n_kv[t];
            if (pv) {
              if (t == 1 || !__all_sync(0xffffffffu, p0_hit)) {
                ok = wait_all(&bars.p_ready[t], (sn[t] + jp) & 1, 6);
                if (!ok) break;
              }
              if (jp == 0 && on[t] > 0) {
                // the first P.V of an item overwrites O_t: the previous item's epilogue must have read it
                ok = wait_all(&bars.o_free[t], (on[t] - 1) & 1, 12);
                if (!ok) break;
              }
            }
            tc_fence_after_sync();
            if (elect_one()) {
              if (pv) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                  umma_ts(tO, tS + kk * 8, vdesc + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv,
                          (jp > 0 || kk > 0) ? 1u : 0u);
                }
                // O_t is complete after its last P.V; the V stage is free after the last P.V reading it
                if (jp == it_.n_kv[t] - 1) umma_commit(smem_u32(&bars.o_done[t]));
                if (t == 1 || !pv1) umma_commit(smem_u32(&bars.v_empty[stp]));
              }
              if (qk) {
                const uint64_t qdesc = umma_smem_desc_sw128(sQ + t * kTileBytes, 16, 1024);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                  const uint64_t off = static_cast<uint64_t>((kk & 3) * 2 + (kk >> 2) * (kHalfBytes >> 4));
                  umma_ss(tS, qdesc + off, kdesc + off, idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&bars.s_full[t]));
                // the K stage is free after the last QK^T that reads it; Q_t after its last QK^T
                if (t == 1 || j >= it_.n_kv[1]) umma_commit(smem_u32(&bars.k_empty[st]));
                if (j == it_.n_kv[t] - 1) umma_commit(smem_u32(&bars.q_empty[t]));
              }
            }
            __syncwarp();
          }
        }
        kc += n_max;
        vc += n_max;
        for (int t = 0; t < 2; ++t) {
          sn[t] += it_.n_kv[t];
          if (it_.n_kv[t] > 0) ++on[t];
        }
      }
    }
  } else if (warp < 4) {
    reg_dealloc<kUtilRegs>();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    reg_alloc<kSoftmaxRegs>();
    const int t = (warp - 4) >> 2;
    const int wq = warp & 3;                     // TMEM lane quarter this warp may touch
    const int r_in_tile = wq * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tbase + lane_base + t * 128;
    const uint32_t tO = tbase + lane_base + 256 + t * 128;
    const float scale = p.scale_log2;
    bool ok = true;
    uint32_t sn = 0;  // tile steps of this tile before the current item
    uint32_t on = 0;  // items of this tile before the current one
    Item it_;
    for (int it = 0; it < n_waves && ok; ++it) {
      if (!get_item<kSplit>(it, p, &it_)) continue;
      const int n_t = it_.n_kv[t];
      if (n_t == 0) continue;
      const int row = it_.q0[t] + r_in_tile;
      int lim = p.Skv - 1;
      if (p.causal) lim = min(lim, row + p.diag_off);
      const int tile_min_lim = p.causal ? min(p.Skv - 1, it_.q0[t] + p.diag_off) : p.Skv - 1;

      float m_ref = -INFINITY;             // exponent reference of this row, in log2 units of the scaled logit
      float l = 0.f;                       // row sum under the current reference

      for (int j = 0; j < n_t && ok; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.s_full[t]), (sn + j) & 1, abortp));
        if (!ok) { if (lane == 0) record_timeout(p.status, 7); break; }
        tc_fence_after_sync();
        const int jk = ((kSplit ? it_.j0 : 0) + j) * kTile;  // first key of this tile
        const bool masked_tile = jk + kTile - 1 > tile_min_lim;
        const int thr = lim - jk;  // columns > thr of this tile are masked for this row

        // The whole 128-wide row is exponentiated at once against the reference left by earlier
        // tiles, so the MUFU starts right after the TMEM load and runs without a gap; the tile's
        // row sum is looked at afterwards.  If it exceeds 2^13 (or is not finite) the rare path
        // takes the true maximum, moves the reference up, rescales what was accumulated under the
        // old one and redoes the tile.
        float e[128];
        {
          uint32_t(&u)[128] = *reinterpret_cast<uint32_t(*)[128]>(e);
          tmem_ld32(tS + 0, *reinterpret_cast<uint32_t(*)[32]>(&u[0]));
          tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&u[32]));
          tmem_ld32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&u[64]));
          tmem_ld32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&u[96]));
          tmem_wait_ld();
        }
        if constexpr (kCap) {
          // cap first, mask afterwards (the reference adds the mask to the capped logits)
#pragma unroll
          for (int i = 0; i < 128; ++i) e[i] = tanh_approx(e[i] * p.cap_in);
        }
        if (masked_tile) {
#pragma unroll
          for (int i = 0; i < 128; ++i) e[i] = (i > thr) ? -INFINITY : e[i];
        }
#ifndef ASUKA_NO_SEED
        if (j == 0) {
          // the first tile of an item has no reference yet: take the tile's true row maximum (the
          // capped and scaled logit is monotone in the raw one) instead of exponentiating blind
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < 128; i += 8) {
            mx4[0] = max3(mx4[0], e[i], e[i + 1]);
            mx4[1] = max3(mx4[1], e[i + 2], e[i + 3]);
            mx4[2] = max3(mx4[2], e[i + 4], e[i + 5]);
            mx4[3] = max3(mx4[3], e[i + 6], e[i + 7]);
          }
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          m_ref = mx > -INFINITY ? mx * (kCap ? p.cap_out : scale) : 0.f;
        }
#endif
        {
          // two logits per FMA instruction (packed f32x2): the softmax warp of a tile runs alone on
          // its scheduler and is bound by the number of instructions it has to issue
          const float mul = kCap ? p.cap_out : scale;
          const float2 mul2 = make_float2(mul, mul), neg_m2 = make_float2(-m_ref, -m_ref);
#ifdef ASUKA_NO_PACKED
          (void)mul2; (void)neg_m2;
#pragma unroll
          for (int i = 0; i < 128; ++i) e[i] = ex2(fmaf(e[i], mul, -m_ref));
#else
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float2 x = __ffma2_rn(make_float2(e[2 * i], e[2 * i + 1]), mul2, neg_m2);
            e[2 * i] = ex2(x.x);
            e[2 * i + 1] = ex2(x.y);
          }
#endif
        }
        // The tile's row sum doubles as the overflow probe: it bounds every term from above, and it
        // is NaN or infinite exactly when some term is.  P is packed
        // to 16 bits right away (the compiler interleaves it with the exponentials), so that only
        // the TMEM store is left once the probe has passed.
        float2 ts4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          ts4[i & 3] = __fadd2_rn(ts4[i & 3], make_float2(e[2 * i], e[2 * i + 1]));
          pk[i] = pack2<kBF16>(e[2 * i], e[2 * i + 1]);
        }
        const float2 ts2 = __fadd2_rn(__fadd2_rn(ts4[0], ts4[1]), __fadd2_rn(ts4[2], ts4[3]));
        float tile_sum = ts2.x + ts2.y;
        const bool need = !(tile_sum <= kRescaleLimit);
        if (__any_sync(0xffffffffu, need)) {
          // ---- rare: the raw logits are still intact in TMEM; take their maximum, 32 columns at a time
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t u[32];
            tmem_ld32(tS + c * 32, u);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = (masked_tile && c * 32 + i > thr) ? -INFINITY : __uint_as_float(u[i]);
              mx = fmaxf(mx, v);
            }
          }
          // the scaled (and capped) logit is monotone in the raw one: transform the maximum
          const float mx2 = kCap ? tanh_approx(mx * p.cap_in) * p.cap_out : mx * scale;
          float alpha = 1.f;
          if (need) {
            alpha = ex2(m_ref - mx2);
            m_ref = mx2;
            l *= alpha;
          }
          if (j > 0) {
            // O_t is the sum over earlier tiles of this work item.  P.V of tile j-1 was issued before
            // QK^T of tile j and the tensor pipe retires in order, so S_t(j) being ready means O_t is
            // complete.
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(tO + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + c * 32, o);
            }
            tmem_wait_st();
          }
          const float mul = kCap ? p.cap_out : scale;
          const float neg_m = -m_ref;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t u[32];
            tmem_ld32(tS + c * 32, u);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float v = __uint_as_float(u[i]);
              if constexpr (kCap) v = tanh_approx(v * p.cap_in);
              v = (masked_tile && c * 32 + i > thr) ? -INFINITY : v;
              e[c * 32 + i] = ex2(fmaf(v, mul, neg_m));
            }
          }
          tile_sum = 0.f;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            tile_sum += e[2 * i] + e[2 * i + 1];
            pk[i] = pack2<kBF16>(e[2 * i], e[2 * i + 1]);
          }
        }
        l += tile_sum;
        tmem_st32(tS, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        if (!ok) break;
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bars.p_ready[t]));
      }
      if (!ok) break;

      // ---- epilogue of the item: O_t / l straight from TMEM to global memory
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.o_done[t]), on & 1, abortp));
      if (!ok) { if (lane == 0) record_timeout(p.status, 9); break; }
      tc_fence_after_sync();
#ifdef ASUKA_REDECODE
      get_item<kSplit>(it, p, &it_);  // (decoded again rather than kept in registers across the key loop)
#endif
      if (kSplit && it_.nparts[t] > 1) {
        // this tile's keys are shared with other items: leave the unnormalised O, the exponent
        // reference and the row sum for the merge (a row that saw no key in this part has l = 0
        // and must not set the scale: its reference goes out as -inf)
        const size_t prow = ((static_cast<size_t>(it_.b) * p.H + it_.h) * p.Sq + row) * p.parts + it_.part;
        float* orow = p.part_o + prow * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (c == 3) {
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars.o_free[t]));
          }
          if (row < p.Sq) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t w[8] = {o[g * 8], o[g * 8 + 1], o[g * 8 + 2], o[g * 8 + 3],
                                     o[g * 8 + 4], o[g * 8 + 5], o[g * 8 + 6], o[g * 8 + 7]};
              st_global_v8(orow + c * 32 + g * 8, w);  // (the workspace rows are 512-byte aligned)
            }
          }
        }
        if (row < p.Sq)
          *reinterpret_cast<float2*>(p.part_ml + prow * 2) = make_float2(l > 0.f ? m_ref : -INFINITY, l);
      } else {
        const float inv_l = 1.f / l;
        uint16_t* orow = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(it_.b) * p.o_sb +
                         static_cast<int64_t>(row) * p.o_ss + static_cast<int64_t>(it_.h) * p.o_sh;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (c == 3) {
            // O_t is in registers: the next item's first P.V may overwrite it
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars.o_free[t]));
          }
          if (row < p.Sq) {
            uint32_t w[16];
#pragma unroll
            for (int g = 0; g < 16; ++g)
              w[g] = pack2<kBF16>(__uint_as_float(o[2 * g]) * inv_l, __uint_as_float(o[2 * g + 1]) * inv_l);
            if (p.out_vec32) {
              st_global_v8(orow + c * 32, *reinterpret_cast<const uint32_t(*)[8]>(&w[0]));
              st_global_v8(orow + c * 32 + 16, *reinterpret_cast<const uint32_t(*)[8]>(&w[8]));
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
            }
          }
        }
        if (p.lse2 != nullptr && row < p.Sq) {
          p.lse2[(static_cast<size_t>(it_.b) * p.H + it_.h) * p.Sq + row] = m_ref + log2f(l);
        }
      }
      sn += n_t;
      ++on;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 512);
  }
}

// Combines the parts of a key-range split.  A warp takes four query rows, lane = four output
// columns: every part's reference, row sum and 512-byte O row are read (they were written moments
// ago and sit in L2) with all loads of the four rows in flight at once -- the kernel is bound by
// that latency, not by the bytes -- scaled to the common reference and added in part order, so the
// result does not depend on which part finished first.
constexpr int kMaxParts = 4;
constexpr int kMergeWarps = 8;
constexpr int kMergeRowsPerWarp = 4;
constexpr int kMergeRows = kMergeWarps * kMergeRowsPerWarp;  // rows per CTA (divides the tile height)
template <bool kBF16>
__global__ void __launch_bounds__(kMergeWarps * 32) attn_merge_kernel(const FwdParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh_count = p.B * p.H;
  const int rb = static_cast<int>(blockIdx.x) / bh_count;  // block of kMergeRows query rows
  const int bh = static_cast<int>(blockIdx.x) % bh_count;
  const int b = bh / p.H, h = bh % p.H;
  const int row0 = rb * kMergeRows + warp * kMergeRowsPerWarp;
  const int q0 = (row0 / kTile) * kTile;
  // the same arithmetic as decode_item: the parts of the 256-row block these rows' tile belongs to
  const int qa = (row0 / (2 * kTile)) * 2 * kTile;
  const int len = (max(kv_tiles_for(qa, p), kv_tiles_for(qa + kTile, p)) + p.parts - 1) / p.parts;
  const int nparts = (kv_tiles_for(q0, p) + len - 1) / len;
  griddep_wait();               // the parts are the output of the kernel ahead
  griddep_launch_dependents();
  if (nparts <= 1) return;      // (one part: the forward kernel wrote the result itself)
  float2 ml[kMergeRowsPerWarp][kMaxParts];
  float4 o[kMergeRowsPerWarp][kMaxParts];
#pragma unroll
  for (int r = 0; r < kMergeRowsPerWarp; ++r) {
    const size_t prow = (static_cast<size_t>(bh) * p.Sq + min(row0 + r, p.Sq - 1)) * p.parts;
#pragma unroll
    for (int q = 0; q < kMaxParts; ++q) {
      if (q < nparts) {
        ml[r][q] = *reinterpret_cast<const float2*>(p.part_ml + (prow + q) * 2);
        o[r][q] = *reinterpret_cast<const float4*>(p.part_o + (prow + q) * 128 + lane * 4);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kMergeRowsPerWarp; ++r) {
    const int row = row0 + r;
    if (row >= p.Sq) break;
    float m = -INFINITY;
#pragma unroll
    for (int q = 0; q < kMaxParts; ++q)
      if (q < nparts) m = fmaxf(m, ml[r][q].x);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kMaxParts; ++q) {
      if (q < nparts) {
        const float w = ml[r][q].x > -INFINITY ? ex2(ml[r][q].x - m) : 0.f;
        l = fmaf(w, ml[r][q].y, l);
        acc.x = fmaf(w, o[r][q].x, acc.x);
        acc.y = fmaf(w, o[r][q].y, acc.y);
        acc.z = fmaf(w, o[r][q].z, acc.z);
        acc.w = fmaf(w, o[r][q].w, acc.w);
      }
    }
    const float inv_l = 1.f / l;
    uint16_t* orow = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(b) * p.o_sb +
                     static_cast<int64_t>(row) * p.o_ss + static_cast<int64_t>(h) * p.o_sh;
    uint2 v;
    v.x = pack2<kBF16>(acc.x * inv_l, acc.y * inv_l);
    v.y = pack2<kBF16>(acc.z * inv_l, acc.w * inv_l);
    *reinterpret_cast<uint2*>(orow + lane * 4) = v;
    if (p.lse2 != nullptr && lane == 0) p.lse2[static_cast<size_t>(bh) * p.Sq + row] = m + log2f(l);
  }
}

}  // namespace

// How many parts the key range of every work item is cut into.  Splitting pays only when the
// launch has fewer items than SMs and the items are long (measured at head counts of 4 to 32 and
// S = 1024 to 4096: the partial results cost about as much L2 traffic again as the inputs); it
// needs workspace for the parts' partial results.
int attn_fwd_parts(const AttnShape& s, int num_sms, size_t ws_bytes) {
  const long long nq_blocks = (s.Sq + 2 * kTile - 1) / (2 * kTile);
  const long long n_items = nq_blocks * s.B * s.H;
  const int max_tiles = (s.Skv + kTile - 1) / kTile;
  int parts = 1;
#ifdef ASUKA_TUNE_ENV
  if (const char* e = getenv("ASUKA_FWD_PARTS")) {
    parts = atoi(e);
    while (parts > 1 && attn_fwd_split_bytes(s, parts) > ws_bytes) parts /= 2;
    return parts;
  }
#endif
  if (n_items < num_sms && max_tiles >= 32) parts = 2 * n_items <= num_sms ? 4 : 2;
  while (parts > 1 && attn_fwd_split_bytes(s, parts) > ws_bytes) parts /= 2;
  return parts;
}

size_t attn_fwd_split_bytes(const AttnShape& s, int parts) {
  if (parts <= 1) return 0;
  const size_t rows = static_cast<size_t>(s.B) * s.H * s.Sq;
  return rows * parts * (128 + 2) * sizeof(float);
}

cudaError_t launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                            void* out, int64_t o_sb, int64_t o_ss, int64_t o_sh, float* lse2,
                            const AttnShape& s, int num_sms, void* split_ws, int parts, cudaStream_t stream) {
  FwdParams p;
  p.B = s.B;
  p.H = s.H;
  p.Sq = s.Sq;
  p.Skv = s.Skv;
  p.causal = s.causal;
  p.diag_off = s.Skv - s.Sq;
  p.nq_blocks = (s.Sq + 2 * kTile - 1) / (2 * kTile);
  p.parts = parts > 1 && split_ws != nullptr ? (parts < kMaxParts ? parts : kMaxParts) : 1;
  p.n_items = p.nq_blocks * s.B * s.H * p.parts;
  p.nq_tiles = (s.Sq + kTile - 1) / kTile;
  {
    const double kv_bytes = 2.0 * s.B * (s.H / (s.group > 0 ? s.group : 1)) * static_cast<double>(s.Skv) * 128 * 2;
#ifdef ASUKA_FWD_NO_UNIT_MAJOR
    p.unit_major = 0;
#else
    p.unit_major = (p.parts == 1 && p.n_items > num_sms && kv_bytes > 96e6) ? 1 : 0;
#endif
  }
#ifdef ASUKA_FWD_NO_PAIR_FAR
  p.pair_far = 0;
#else
  p.pair_far = (p.parts == 1 && s.causal && p.n_items <= num_sms && p.nq_tiles >= 4) ? 1 : 0;
#endif
  p.group = s.group;
  p.scale_log2 = s.softmax_scale * 1.4426950408889634f;
  p.cap_in = s.softcap > 0.f ? s.softmax_scale / s.softcap : 0.f;
  p.cap_out = s.softcap * 1.4426950408889634f;
  p.lse2 = lse2;
  p.out = out;
  p.o_sb = o_sb;
  p.o_ss = o_ss;
  p.o_sh = o_sh;
  p.out_vec32 = (reinterpret_cast<uintptr_t>(out) % 32 == 0 && o_sb % 16 == 0 && o_ss % 16 == 0 && o_sh % 16 == 0) ? 1 : 0;
  p.status = device_status_words();
  p.part_o = static_cast<float*>(split_ws);
  p.part_ml = p.part_o + static_cast<size_t>(s.B) * s.H * s.Sq * p.parts * 128;
  const dim3 grid(static_cast<unsigned>(p.n_items < num_sms ? p.n_items : num_sms));
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, FwdParams);
  if (p.parts > 1) {
    if (s.softcap > 0.f) kern = s.bf16 ? attn_fwd_kernel<true, true, true> : attn_fwd_kernel<false, true, true>;
    else kern = s.bf16 ? attn_fwd_kernel<true, false, true> : attn_fwd_kernel<false, false, true>;
  } else {
    if (s.softcap > 0.f) kern = s.bf16 ? attn_fwd_kernel<true, true, false> : attn_fwd_kernel<false, true, false>;
    else kern = s.bf16 ? attn_fwd_kernel<true, false, false> : attn_fwd_kernel<false, false, false>;
  }
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes);
  if (e != cudaSuccess) return e;
  e = check_register_budget(reinterpret_cast<const void*>(kern), kThreads, 128 * kUtilRegs + 256 * kSoftmaxRegs);
  if (e != cudaSuccess) return e;
  e = launch_dependent(kern, grid, dim3(kThreads), kSmemBytes, stream, mq, mk, mv, p);
  count_launch();
  if (e != cudaSuccess || p.parts == 1) return e;
  const dim3 mgrid(static_cast<unsigned>((s.Sq + kMergeRows - 1) / kMergeRows) * s.B * s.H);
  e = launch_dependent(s.bf16 ? attn_merge_kernel<true> : attn_merge_kernel<false>, mgrid, dim3(kMergeWarps * 32), 0,
                       stream, p);
  count_launch();
  return e;
}

}  // namespace asuka
