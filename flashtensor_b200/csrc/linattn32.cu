// Linear attention at head_dim 32 in f32: the attention core of the reference's SimA and EA
// benchmark programs at their own shapes (bench/sima.mlir:13-17, bench/ea.mlir:13-17:
// tensor<64x4x784x32xf32>), between the QKV projection and the output projection.
//
//   SimA  out = (Q / sum_n|Q|) . ((K / sum_n|K|)^T . V)      (normalisations over the sequence n)
//   EA    out = softmax_d(Q)   . (softmax_n(K)^T . V)
//
// With 32 features the two products are 2 flops per byte moved, far too few for tensor-core tiles:
// plain CUDA-core code with coalesced accesses.  One CTA per (batch, head); every warp streams
// rows n = w, w + 8, ... of the [N, 32] slices with lane = feature (one 128-byte row per load,
// sixteen rows in flight), three times: column statistics, the 32 x 32 product K'^T V, then the
// output rows.  In the two products a lane keeps one column of the 32 x 32 matrix in registers and
// the other operand's row is broadcast through a per-warp shared-memory buffer with 16-byte loads;
// the multiply-adds are the packed two-wide f32 FMAs of sm_100.  Every sum runs in a fixed order,
// so results are reproducible.  What bounds it is the latency of the row loads: a (batch, head) is
// one dependent chain of three passes, and 256 of them give a B200 only 16 warps per SM, each one
// step of eight rows ahead.  Splitting a (batch, head) over a cluster of 2 or 4 CTAs was measured
// and is slower.
#include "kernels.h"

namespace asuka {
namespace {

constexpr int kD = 32;
constexpr int kWarps = 8;
constexpr int kUnroll = 8;  // rows of a warp per step (twice as many are in flight)

__device__ __forceinline__ float exp_fast(float x) {  // e^x
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// acc[d] += row[d] * x for d = 0..31 (acc as 16 pairs), `row` a 32-float shared-memory buffer
__device__ __forceinline__ void axpy_row(float2 (&acc)[kD / 2], const float* row, float x) {
  const float2 xx = make_float2(x, x);
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 r = *reinterpret_cast<const float4*>(row + g * 4);
    acc[g * 2 + 0] = __ffma2_rn(make_float2(r.x, r.y), xx, acc[g * 2 + 0]);
    acc[g * 2 + 1] = __ffma2_rn(make_float2(r.z, r.w), xx, acc[g * 2 + 1]);
  }
}

template <bool kEA>
__global__ void __launch_bounds__(kWarps * 32) linattn32_kernel(const LinAttn32Args a) {
  __shared__ __align__(16) float row_s[kWarps][kUnroll][kD];  // per warp: rows being broadcast
  __shared__ __align__(16) float m_part[kWarps / 2][kD][kD];  // partial K'^T V, four warps at a time
  __shared__ __align__(16) float m_s[kD][kD];                 // M' = normalised K'^T V, [d][e]
  __shared__ float red[2][kWarps][kD];
  __shared__ float col_a[kD], col_b[kD];  // EA: column maximum, denominator; SimA: sum|K|, sum|Q|

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
  const float* q = a.q + static_cast<int64_t>(b) * a.q_sb + static_cast<int64_t>(h) * a.q_sh + lane;
  const float* k = a.k + static_cast<int64_t>(b) * a.k_sb + static_cast<int64_t>(h) * a.k_sh + lane;
  const float* v = a.v + static_cast<int64_t>(b) * a.v_sb + static_cast<int64_t>(h) * a.v_sh + lane;
  float* out = a.out + static_cast<int64_t>(b) * a.o_sb + static_cast<int64_t>(h) * a.o_sh + lane;
  constexpr int kStep = kWarps * kUnroll;  // rows all warps take per step

  // ---- pass 1: column statistics over the sequence
  {
    float s0 = kEA ? -INFINITY : 0.f, s1 = 0.f;
    for (int n0 = warp; n0 < a.N; n0 += 2 * kStep) {
      float kv[2 * kUnroll], qv[kEA ? 1 : 2 * kUnroll];
#pragma unroll
      for (int u = 0; u < 2 * kUnroll; ++u) {
        const int n = n0 + u * kWarps;
        kv[u] = n < a.N ? __ldg(k + static_cast<int64_t>(n) * a.k_sn) : (kEA ? -INFINITY : 0.f);
        if constexpr (!kEA) qv[u] = n < a.N ? __ldg(q + static_cast<int64_t>(n) * a.q_sn) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 2 * kUnroll; ++u) {
        if constexpr (kEA) {
          s0 = fmaxf(s0, kv[u]);
        } else {
          s0 += fabsf(kv[u]);
          s1 += fabsf(qv[u]);
        }
      }
    }
    red[0][warp][lane] = s0;
    red[1][warp][lane] = s1;
    __syncthreads();
    if (tid < kD) {
      float r0 = red[0][0][tid], r1 = red[1][0][tid];
      for (int w = 1; w < kWarps; ++w) {
        r0 = kEA ? fmaxf(r0, red[0][w][tid]) : r0 + red[0][w][tid];
        r1 += red[1][w][tid];
      }
      col_a[tid] = r0;
      col_b[tid] = r1;
    }
    __syncthreads();
  }

  // ---- pass 2: M[d][e] = sum_n K'[n][d] V[n][e], K' = exp(K - column maximum) (EA) or K (SimA).
  // Lane e keeps column e of this warp's partial M; the K' row is broadcast through row_s.
  {
    float2 acc[kD / 2];
#pragma unroll
    for (int d = 0; d < kD / 2; ++d) acc[d] = make_float2(0.f, 0.f);
    float zsum = 0.f;  // EA: column sum of K' for feature `lane` over this warp's rows
    const float cm = kEA ? col_a[lane] : 0.f;
    // software pipeline: the rows of the next step are in flight while this step's FMAs run
    float kn[kUnroll], vn[kUnroll];
    auto fetch = [&](int n0) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int n = n0 + u * kWarps;
        kn[u] = n < a.N ? __ldg(k + static_cast<int64_t>(n) * a.k_sn) : (kEA ? -INFINITY : 0.f);
        vn[u] = n < a.N ? __ldg(v + static_cast<int64_t>(n) * a.v_sn) : 0.f;
      }
    };
    fetch(warp);
    for (int n0 = warp; n0 < a.N; n0 += kStep) {
      float vv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        float kv = kn[u];
        vv[u] = vn[u];
        if constexpr (kEA) {
          kv = exp_fast(kv - cm);  // rows past the end were loaded as -inf: they give 0
          zsum += kv;
        }
        row_s[warp][u][lane] = kv;
      }
      fetch(n0 + kStep);
      __syncwarp();
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) axpy_row(acc, row_s[warp][u], vv[u]);
      __syncwarp();
    }
    // fixed-order reduction over the warps, four at a time through shared memory
    red[0][warp][lane] = zsum;
    float total[kD];
#pragma unroll
    for (int d = 0; d < kD; ++d) total[d] = 0.f;
#pragma unroll
    for (int round = 0; round < 2; ++round) {
      if ((warp >> 2) == round) {
#pragma unroll
        for (int d = 0; d < kD / 2; ++d) {
          m_part[warp & 3][2 * d][lane] = acc[d].x;
          m_part[warp & 3][2 * d + 1][lane] = acc[d].y;
        }
      }
      __syncthreads();
      if (warp == 0) {
#pragma unroll
        for (int w = 0; w < kWarps / 2; ++w) {
#pragma unroll
          for (int d = 0; d < kD; ++d) total[d] += m_part[w][d][lane];
        }
      }
      __syncthreads();
    }
    if (warp == 0) {
      if constexpr (kEA) {
        float z = 0.f;
        for (int w = 0; w < kWarps; ++w) z += red[0][w][lane];
        col_b[lane] = z;
      }
      __syncwarp();
#pragma unroll
      for (int d = 0; d < kD; ++d) {
        const float inv = kEA ? 1.f / col_b[d] : 1.f / (col_a[d] * col_b[d]);
        m_s[d][lane] = total[d] * inv;
      }
    }
    __syncthreads();
  }

  // ---- pass 3: out[n][e] = sum_d Qn[n][d] M'[d][e]; lane e keeps column e of M' in registers
  {
    float2 mcol[kD / 2];
#pragma unroll
    for (int d = 0; d < kD / 2; ++d) mcol[d] = make_float2(m_s[2 * d][lane], m_s[2 * d + 1][lane]);
    float qn[kUnroll];
    auto fetch_q = [&](int n0) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int n = n0 + u * kWarps;
        qn[u] = n < a.N ? __ldg(q + static_cast<int64_t>(n) * a.q_sn) : 0.f;
      }
    };
    fetch_q(warp);
    for (int n0 = warp; n0 < a.N; n0 += kStep) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        float qv = qn[u];
        if constexpr (kEA) {
          const float e = exp_fast(qv - warp_max(qv));
          qv = e / warp_sum(e);
        }
        row_s[warp][u][lane] = qv;
      }
      fetch_q(n0 + kStep);
      __syncwarp();
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int n = n0 + u * kWarps;
        float2 o2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 r = *reinterpret_cast<const float4*>(&row_s[warp][u][g * 4]);
          o2 = __ffma2_rn(make_float2(r.x, r.y), mcol[g * 2 + 0], o2);
          o2 = __ffma2_rn(make_float2(r.z, r.w), mcol[g * 2 + 1], o2);
        }
        if (n < a.N) out[static_cast<int64_t>(n) * a.o_sn] = o2.x + o2.y;
      }
      __syncwarp();
    }
  }
}

}  // namespace

cudaError_t launch_linattn32(const LinAttn32Args& a, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(a.B) * a.H);
  if (a.ea) linattn32_kernel<true><<<grid, kWarps * 32, 0, stream>>>(a);
  else linattn32_kernel<false><<<grid, kWarps * 32, 0, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

}  // namespace asuka
