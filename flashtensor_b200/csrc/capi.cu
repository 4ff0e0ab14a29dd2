// C-ABI layer: argument validation, tensor-map construction, launch sequencing.
// Declarations and the reference interfaces they replace are in include/asuka_b200.h.
#include <atomic>
#include <cmath>
#include <cstring>

#include "../../include/asuka_b200.h"
#include "kernels.h"
#include "tma_host.h"

namespace asuka {

__device__ uint32_t g_status_words[4];
static std::atomic<uint64_t> g_launches{0};

uint32_t* device_status_words() {
  // one address per device; cached per device id (devices are few)
  static uint32_t* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<uint32_t*>(p);
  }
  return cache[dev];
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {

constexpr int kHeadDim = 128;

int check_arch() {
  static int cached[64];
  static bool have[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ASUKA_ERR_CUDA;
  if (dev < 0 || dev >= 64) return ASUKA_ERR_CUDA;
  if (!have[dev]) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return ASUKA_ERR_CUDA;
    cached[dev] = major;
    have[dev] = true;
  }
  return cached[dev] == 10 ? ASUKA_OK : ASUKA_ERR_UNSUPPORTED_ARCH;
}

bool is_16bit(int dt) { return dt == ASUKA_F16 || dt == ASUKA_BF16; }

// [B,S,H,128] 16-bit tensor usable as a TMA source/destination
int check_bshd(const asuka_tensor& t, int dtype) {
  if (t.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (t.dtype != dtype) return ASUKA_ERR_BAD_DTYPE;
  if (t.ndim != 4) return ASUKA_ERR_BAD_SHAPE;
  for (int i = 0; i < 4; ++i)
    if (t.shape[i] <= 0) return ASUKA_ERR_BAD_SHAPE;
  if (t.shape[3] != kHeadDim) return ASUKA_ERR_BAD_SHAPE;
  if (t.shape[0] > 65535 || t.shape[2] > 65535 || t.shape[1] > (1 << 24)) return ASUKA_ERR_TOO_LARGE;
  if (t.stride[3] != 1) return ASUKA_ERR_BAD_STRIDE;
  for (int i = 0; i < 3; ++i) {
    if (t.stride[i] <= 0 || (t.stride[i] % 8) != 0) return ASUKA_ERR_BAD_STRIDE;
  }
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return ASUKA_ERR_MISALIGNED;
  return ASUKA_OK;
}

// contiguous f32 / i32 tensor of the given shape
int check_dense(const asuka_tensor& t, int dtype, int ndim, const int64_t* shape) {
  if (t.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (t.dtype != dtype) return ASUKA_ERR_BAD_DTYPE;
  if (t.ndim != ndim) return ASUKA_ERR_BAD_SHAPE;
  int64_t expect = 1;
  for (int i = ndim - 1; i >= 0; --i) {
    if (t.shape[i] != shape[i]) return ASUKA_ERR_BAD_SHAPE;
    if (t.shape[i] != 1 && t.stride[i] != expect) return ASUKA_ERR_BAD_STRIDE;
    expect *= shape[i];
  }
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return ASUKA_ERR_MISALIGNED;
  return ASUKA_OK;
}

int make_map(CUtensorMap* m, const asuka_tensor& t) {
  int r = tma_host::make_bshd_map(m, t.ptr, t.dtype == ASUKA_BF16, t.shape[0], t.shape[1], t.shape[2],
                                  t.shape[3], t.stride[0], t.stride[1], t.stride[2], 128);
  return r == 0 ? ASUKA_OK : ASUKA_ERR_CUDA;
}

struct QKV {
  AttnShape s;
  int dtype;
};

// shared validation of q/k(/v/out): shapes agree, causal needs Skv >= Sq
int check_qk(const asuka_tensor& q, const asuka_tensor& k, float scale, int causal, QKV* o) {
  if (!is_16bit(q.dtype)) return q.ptr == nullptr ? ASUKA_ERR_NULL_POINTER : ASUKA_ERR_BAD_DTYPE;
  int r;
  if ((r = check_bshd(q, q.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(k, q.dtype)) != ASUKA_OK) return r;
  if (k.shape[0] != q.shape[0] || k.shape[2] != q.shape[2]) return ASUKA_ERR_BAD_SHAPE;
  if (causal && k.shape[1] < q.shape[1]) return ASUKA_ERR_BAD_SHAPE;
  if (std::isnan(scale) || std::isinf(scale)) return ASUKA_ERR_BAD_ARGUMENT;
  o->dtype = q.dtype;
  o->s.B = static_cast<int>(q.shape[0]);
  o->s.Sq = static_cast<int>(q.shape[1]);
  o->s.H = static_cast<int>(q.shape[2]);
  o->s.Skv = static_cast<int>(k.shape[1]);
  o->s.causal = causal ? 1 : 0;
  o->s.softmax_scale = scale > 0.f ? scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
  o->s.bf16 = q.dtype == ASUKA_BF16;
  return ASUKA_OK;
}

int map_cuda(cudaError_t e) { return e == cudaSuccess ? ASUKA_OK : ASUKA_ERR_CUDA; }

int attn_fwd_impl(const asuka_attn_params* p, float* lse_override, cudaStream_t stream) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  QKV c;
  int r;
  if ((r = check_qk(p->q, p->k, p->softmax_scale, p->causal, &c)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->v, c.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->out, c.dtype)) != ASUKA_OK) return r;
  for (int i = 0; i < 4; ++i) {
    if (p->v.shape[i] != p->k.shape[i] || p->out.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
  }
  float* lse = lse_override;
  if (lse == nullptr && p->lse.ptr != nullptr) {
    const int64_t shp[3] = {c.s.B, c.s.H, c.s.Sq};
    if ((r = check_dense(p->lse, ASUKA_F32, 3, shp)) != ASUKA_OK) return r;
    lse = static_cast<float*>(p->lse.ptr);
  }
  if ((r = check_arch()) != ASUKA_OK) return r;
  CUtensorMap mq, mk, mv, mo;
  if ((r = make_map(&mq, p->q)) || (r = make_map(&mk, p->k)) || (r = make_map(&mv, p->v)) ||
      (r = make_map(&mo, p->out)))
    return r;
  return map_cuda(launch_attn_fwd(mq, mk, mv, mo, lse, c.s, stream));
}

}  // namespace
}  // namespace asuka

using namespace asuka;

extern "C" {

int asuka_b200_version(void) { return 100; }

const char* asuka_b200_strerror(int status) {
  switch (status) {
    case ASUKA_OK: return "ok";
    case ASUKA_ERR_NULL_POINTER: return "null pointer";
    case ASUKA_ERR_BAD_DTYPE: return "unsupported or mismatched dtype";
    case ASUKA_ERR_BAD_SHAPE: return "bad shape";
    case ASUKA_ERR_BAD_STRIDE: return "bad stride (innermost must be 1, others multiples of 8 elements)";
    case ASUKA_ERR_MISALIGNED: return "pointer not 16-byte aligned";
    case ASUKA_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case ASUKA_ERR_UNSUPPORTED_ARCH: return "device is not sm_100";
    case ASUKA_ERR_CUDA: return "CUDA runtime error";
    case ASUKA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    case ASUKA_ERR_BAD_ARGUMENT: return "bad scalar argument";
    case ASUKA_ERR_TOO_LARGE: return "size beyond the supported maximum";
    default: return "unknown status";
  }
}

uint64_t asuka_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int asuka_b200_device_status(uint32_t* out) {
  if (out == nullptr) return ASUKA_ERR_NULL_POINTER;
  uint32_t w[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return ASUKA_ERR_CUDA;
  if (cudaMemcpyFromSymbol(w, g_status_words, sizeof(w)) != cudaSuccess) return ASUKA_ERR_CUDA;
  out[0] = w[0];
  out[1] = w[1];
  if (w[0] != 0) {
    const uint32_t z[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status_words, z, sizeof(z)) != cudaSuccess) return ASUKA_ERR_CUDA;
    return ASUKA_ERR_DEVICE_TIMEOUT;
  }
  return ASUKA_OK;
}

int asuka_b200_attn_fwd(const asuka_attn_params* p, asuka_stream stream) {
  return attn_fwd_impl(p, nullptr, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
