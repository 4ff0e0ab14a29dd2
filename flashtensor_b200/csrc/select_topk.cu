// Heavy-hitter selection: the indices of the k largest per-key scores of every (batch, head) row,
// written in ascending index order.  The reference stops at the scores (it has no top-k, sort or
// eviction code); the rules are the benchmark configuration's:
//   TOPK          k largest keys, equal keys -> lower index first
//   TOPK_RECENT   k largest among positions [0, S-recent), then the last `recent` positions (H2O)
//   ROCO          key = (mean, std) with mean = sum/n_j, std = sqrt(max(sumsq/n_j - mean^2, 0)),
//                 n_j = q_len - max(0, j - (S - q_len)) (causal) or q_len (unmasked); larger mean
//                 first, then larger std, then lower index; mean and std are optional outputs
// One CTA per row.  Keys are mapped to order-preserving unsigned integers and kept in shared
// memory; an MSB-first radix select (11 bits per pass: three passes for 32-bit keys, six for 64-bit
// ones; shared-memory atomics on a 2048-bin histogram, warp-aggregated where equal digits are
// common) finds the k-th largest key exactly, then an ordered block scan compacts the kept
// indices.  Everything is
// integer work on exact keys, so the result is deterministic.
#include "../../include/asuka_b200.h"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace asuka {
namespace {

constexpr int kSelThreads = 1024;

__device__ __forceinline__ uint32_t mono_f32(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename KeyT>
__device__ __forceinline__ KeyT make_key(const SelectArgs& a, const float* srow, const float* qrow,
                                         int j);

template <>
__device__ __forceinline__ uint32_t make_key<uint32_t>(const SelectArgs&, const float* srow,
                                                       const float*, int j) {
  return mono_f32(srow[j]);
}
template <>
__device__ __forceinline__ uint64_t make_key<uint64_t>(const SelectArgs& a, const float* srow,
                                                       const float* qrow, int j) {
  // IEEE-exact, unfused f32 arithmetic so that the keys equal a plain f32 CPU evaluation bit for bit
  const float n = static_cast<float>(a.all_rows ? a.q_len : a.q_len - max(0, j - (a.S - a.q_len)));
  const float mean = __fdiv_rn(srow[j], n);
  const float var = fmaxf(__fsub_rn(__fdiv_rn(qrow[j], n), __fmul_rn(mean, mean)), 0.f);
  const float sd = __fsqrt_rn(var);
  if (a.mean != nullptr) a.mean[static_cast<size_t>(blockIdx.x) * a.S + j] = mean;
  if (a.std != nullptr) a.std[static_cast<size_t>(blockIdx.x) * a.S + j] = sd;
  return (static_cast<uint64_t>(mono_f32(mean)) << 32) | mono_f32(sd);
}

constexpr int kDigitBits = 11;
constexpr int kBins = 1 << kDigitBits;  // two bins per thread

template <typename KeyT>
__global__ void __launch_bounds__(kSelThreads, 1) select_kernel(const SelectArgs a) {
  extern __shared__ __align__(16) uint8_t sel_smem[];
  KeyT* keys = reinterpret_cast<KeyT*>(sel_smem);
  __shared__ uint32_t hist[kBins];
  __shared__ uint32_t warp_sum[32];
  __shared__ unsigned long long warp_tot[32];
  __shared__ KeyT s_prefix;
  __shared__ uint32_t s_k;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const float* srow = a.score + static_cast<size_t>(row) * a.S;
  const float* qrow = a.score_sq ? a.score_sq + static_cast<size_t>(row) * a.S : nullptr;
  const int n_out = a.k_keep + (a.mode == ASUKA_SELECT_TOPK_RECENT ? a.recent : 0);
  int32_t* out = a.idx + static_cast<size_t>(row) * n_out;
  const int ncand = a.mode == ASUKA_SELECT_TOPK_RECENT ? a.S - a.recent : a.S;

  // (launched as a programmatic dependent: the scores are the output of the kernel ahead)
  sm100::griddep_wait();
  sm100::griddep_launch_dependents();
  if (a.n_chunks > 0) {
    // the column pass left partial sums per query range: add them in range order and write the
    // scores (every thread later reads back only what it wrote itself: same stride)
    const size_t n = static_cast<size_t>(a.rows) * a.S, off = static_cast<size_t>(row) * a.S;
    float* sw = const_cast<float*>(srow);
    float* qw = const_cast<float*>(qrow);
    for (int j = tid; j < a.S; j += kSelThreads) {
      float s1 = 0.f, s2 = 0.f;
      for (int c = 0; c < a.n_chunks; ++c) {
        s1 += a.part[c * n + off + j];
        if (a.part_sq != nullptr) s2 += a.part_sq[c * n + off + j];
      }
      sw[j] = s1;
      if (a.part_sq != nullptr) qw[j] = s2;
    }
  }
  for (int j = tid; j < ncand; j += kSelThreads) keys[j] = make_key<KeyT>(a, srow, qrow, j);
  hist[tid] = 0;
  hist[tid + kSelThreads] = 0;
  __syncthreads();

  constexpr int kKeyBits = static_cast<int>(sizeof(KeyT)) * 8;
  KeyT prefix = 0, mask = 0;
  uint32_t k = static_cast<uint32_t>(a.k_keep);
  for (int hi = kKeyBits; hi > 0; hi -= kDigitBits) {
    // this pass looks at bits [lo, hi); the last pass of a key may be narrower than 11 bits
    const int lo = hi > kDigitBits ? hi - kDigitBits : 0;
    const uint32_t dmask = (1u << (hi - lo)) - 1u;
    for (int base = 0; base < ncand; base += kSelThreads) {
      const int j = base + tid;
      bool in = false;
      uint32_t digit = 0;
      if (j < ncand) {
        const KeyT key = keys[j];
        in = (key & mask) == prefix;
        digit = static_cast<uint32_t>(key >> lo) & dmask;
      }
      const uint32_t act = __ballot_sync(0xffffffffu, in);
      if (act == 0u) continue;
      if constexpr (sizeof(KeyT) == 8) {
        // composite (mean, std) keys share most of their leading bits: aggregate equal digits in
        // the warp before touching the histogram
        if (in) {
          const uint32_t peers = __match_any_sync(act, digit);
          if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], __popc(peers));
        }
      } else {
        // scores spread over the bins, so plain atomics rarely collide; the one degenerate case
        // worth a check is a warp whose live keys all carry the same digit
        const int leader = __ffs(act) - 1;
        const uint32_t d0 = __shfl_sync(0xffffffffu, digit, leader);
        if (__all_sync(0xffffffffu, !in || digit == d0)) {
          if (lane == leader) atomicAdd(&hist[d0], __popc(act));
        } else if (in) {
          atomicAdd(&hist[digit], 1u);
        }
      }
    }
    __syncthreads();
    // Find the digit d with count(digits > d) < k <= count(digits >= d).  Thread t owns bins 2t and
    // 2t + 1; suffix sums run over the lanes of a warp, then over the 32 warps.
    const uint32_t c0 = hist[2 * tid], c1 = hist[2 * tid + 1];
    hist[2 * tid] = 0;      // (cleared for the next pass; nobody else reads these two bins)
    hist[2 * tid + 1] = 0;
    const uint32_t mine = c0 + c1;
    uint32_t incl = mine;   // sum over lanes >= this one of this warp
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t v = __shfl_down_sync(0xffffffffu, incl, off);
      if (lane + off < 32) incl += v;
    }
    if (lane == 0) warp_sum[warp] = incl;
    __syncthreads();
    uint32_t higher = 0;    // keys in the bins of all higher warps
    {
      const uint32_t v = (lane > warp) ? warp_sum[lane] : 0u;
      higher = __reduce_add_sync(0xffffffffu, v);
    }
    const uint32_t above = higher + incl - mine;  // keys with a digit above this thread's two bins
    if (above < k && k <= above + mine) {
      uint32_t r = k - above;
      int d = 2 * tid + 1;
      if (c1 < r) {
        r -= c1;
        d = 2 * tid;
      }
      s_prefix = prefix | (static_cast<KeyT>(d) << lo);
      s_k = r;
    }
    __syncthreads();
    prefix = s_prefix;
    k = s_k;
    mask |= static_cast<KeyT>(dmask) << lo;
  }
  // prefix is now the k-th largest key T; k of the keys equal to T are kept, lowest index first.

  const int chunk = (ncand + kSelThreads - 1) / kSelThreads;
  const int lo = min(tid * chunk, ncand), hi = min(lo + chunk, ncand);
  uint32_t cg = 0, ce = 0;
  for (int j = lo; j < hi; ++j) {
    const KeyT key = keys[j];
    cg += key > prefix;
    ce += key == prefix;
  }
  // ordered exclusive scan of (cg, ce) over the block, both packed into one 64-bit word
  const unsigned long long mine = (static_cast<unsigned long long>(cg) << 32) | ce;
  unsigned long long incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const unsigned long long t = warp_tot[lane];
    unsigned long long w = t;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long v = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += v;
    }
    warp_tot[lane] = w - t;
  }
  __syncthreads();
  const unsigned long long excl = warp_tot[warp] + incl - mine;
  uint32_t pg = static_cast<uint32_t>(excl >> 32), pe = static_cast<uint32_t>(excl & 0xffffffffu);
  for (int j = lo; j < hi; ++j) {
    const KeyT key = keys[j];
    if (key > prefix) {
      out[pg + min(pe, k)] = j;
      ++pg;
    } else if (key == prefix) {
      if (pe < k) out[pg + pe] = j;
      ++pe;
    }
  }
  if (a.mode == ASUKA_SELECT_TOPK_RECENT) {
    for (int j = tid; j < a.recent; j += kSelThreads) out[a.k_keep + j] = a.S - a.recent + j;
  }
}

}  // namespace

cudaError_t launch_select(const SelectArgs& a, cudaStream_t stream) {
  const bool wide = a.mode == ASUKA_SELECT_ROCO;
  const size_t smem = static_cast<size_t>(a.S) * (wide ? 8 : 4);
  cudaError_t e;
  if (wide) {
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(select_kernel<uint64_t>), static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    e = launch_dependent(select_kernel<uint64_t>, dim3(a.rows), dim3(kSelThreads), smem, stream, a);
  } else {
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(select_kernel<uint32_t>), static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    e = launch_dependent(select_kernel<uint32_t>, dim3(a.rows), dim3(kSelThreads), smem, stream, a);
  }
  count_launch();
  return e;
}

}  // namespace asuka
