// Small per-key score post-processing kernels.
//
// pool_scores: SnapKV's smoothing of the per-key scores, F.avg_pool1d(score, kernel_size,
// padding=kernel_size/2, stride=1) along the key axis (cases/kernels/snapkv.py:35-38): a zero-padded
// moving sum divided by kernel_size (padding counts towards the divisor, PyTorch's default).
#include "kernels.h"
#include "sm100_ptx.cuh"
//
// gather_kv: KV-cache compaction after a selection, k_out[b, n, h, :] = k[b, idx[b, h, n], h, :]
// (and v alike): 256-byte rows moved with 16-byte loads and stores, 16 lanes per row.

namespace asuka {
namespace {

// Self-test of the time-out path every pipeline kernel relies on: one thread waits, through the
// same bounded wait, on a barrier nothing will ever complete, gives up after `limit_ns` and leaves
// the same record a stuck pipeline would.  The kernel returns normally and the context stays usable.
__global__ void wait_selftest_kernel(uint32_t* status, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_s;
  abort_s = 0;
  sm100::mbar_init(sm100::smem_u32(&bar), 1);
  sm100::mbar_fence_init();
  volatile uint32_t* abortp = &abort_s;
  if (!sm100::mbar_wait(sm100::smem_u32(&bar), 0, abortp, limit_ns)) {
    atomicAdd(&status[0], 1u);
    status[1] = 99;  // site id of the self-test
  }
}

__global__ void __launch_bounds__(256) pool_scores_kernel(const float* __restrict__ in,
                                                          float* __restrict__ out, int rows, int S,
                                                          int ksize) {
  const int row = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows || j >= S) return;
  const float* r = in + static_cast<size_t>(row) * S;
  const int half = ksize / 2;
  float acc = 0.f;
  for (int d = -half; d <= half; ++d) {
    const int jj = j + d;
    if (jj >= 0 && jj < S) acc += r[jj];
  }
  out[static_cast<size_t>(row) * S + j] = acc / static_cast<float>(ksize);
}

// group_mean: grouped-query attention's per-key score, the mean over the query heads of a group
// (cases/attn_h2o.py:42-46), summed in head order.
__global__ void __launch_bounds__(256) group_mean_kernel(const float* __restrict__ in,
                                                         float* __restrict__ out, int rows, int group,
                                                         int S) {
  const int row = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows || j >= S) return;
  float acc = 0.f;
  for (int g = 0; g < group; ++g) acc += in[(static_cast<size_t>(row) * group + g) * S + j];
  out[static_cast<size_t>(row) * S + j] = acc / static_cast<float>(group);
}

__global__ void __launch_bounds__(256) gather_kv_kernel(GatherArgs a) {
  const int h = blockIdx.y, b = blockIdx.z;
  const int lane16 = threadIdx.x & 15;
  const int row_in_block = threadIdx.x >> 4;  // 16 rows per block step
  const int32_t* idx = a.idx + (static_cast<size_t>(b) * a.H + h) * a.n;
  for (int n = blockIdx.x * 16 + row_in_block; n < a.n; n += gridDim.x * 16) {
    int src = idx[n];
    src = src < 0 ? 0 : (src >= a.S ? a.S - 1 : src);  // indices are trusted to be in range; never read outside
    const size_t in_off = static_cast<size_t>(b) * a.in_sb + static_cast<size_t>(src) * a.in_ss +
                          static_cast<size_t>(h) * a.in_sh;
    const size_t out_off = static_cast<size_t>(b) * a.out_sb + static_cast<size_t>(n) * a.out_ss +
                           static_cast<size_t>(h) * a.out_sh;
    const uint4 kv = reinterpret_cast<const uint4*>(a.k + in_off)[lane16];
    const uint4 vv = reinterpret_cast<const uint4*>(a.v + in_off)[lane16];
    reinterpret_cast<uint4*>(a.k_out + out_off)[lane16] = kv;
    reinterpret_cast<uint4*>(a.v_out + out_off)[lane16] = vv;
  }
}

}  // namespace

cudaError_t launch_wait_selftest(uint64_t limit_ns, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 1, 0, stream>>>(device_status_words(), limit_ns);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_gather_kv(const GatherArgs& a, cudaStream_t stream) {
  int bx = (a.n + 15) / 16;
  if (bx > 64) bx = 64;
  const dim3 grid(bx, a.H, a.B);
  gather_kv_kernel<<<grid, 256, 0, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_group_mean(const float* in, float* out, int rows, int group, int S, cudaStream_t stream) {
  const dim3 grid((S + 255) / 256, rows);
  group_mean_kernel<<<grid, 256, 0, stream>>>(in, out, rows, group, S);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pool_scores(const float* in, float* out, int rows, int S, int ksize,
                               cudaStream_t stream) {
  const dim3 grid((S + 255) / 256, rows);
  pool_scores_kernel<<<grid, 256, 0, stream>>>(in, out, rows, S, ksize);
  count_launch();
  return cudaGetLastError();
}

}  // namespace asuka
