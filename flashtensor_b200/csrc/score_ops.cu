// Small per-key score post-processing kernels.
//
// pool_scores: SnapKV's smoothing of the per-key scores, F.avg_pool1d(score, kernel_size,
// padding=kernel_size/2, stride=1) along the key axis (cases/kernels/snapkv.py:35-38): a zero-padded
// moving sum divided by kernel_size (padding counts towards the divisor, PyTorch's default).
#include "kernels.h"

namespace asuka {
namespace {

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

}  // namespace

cudaError_t launch_pool_scores(const float* in, float* out, int rows, int S, int ksize,
                               cudaStream_t stream) {
  const dim3 grid((S + 255) / 256, rows);
  pool_scores_kernel<<<grid, 256, 0, stream>>>(in, out, rows, S, ksize);
  count_launch();
  return cudaPeekAtLastError();
}

}  // namespace asuka
