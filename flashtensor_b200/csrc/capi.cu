// C-ABI layer: argument validation, tensor-map construction, launch sequencing.
// Declarations and the reference interfaces they replace are in include/asuka_b200.h.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "../../include/asuka_b200.h"
#include "kernels.h"
#include "tma_host.h"

namespace asuka {

__device__ uint32_t g_status_words[4];
static std::atomic<uint64_t> g_launches{0};

uint32_t* device_status_words() {
  // one address per device; cached per device id (devices are few)
  static std::mutex mu;
  static uint32_t* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<uint32_t*>(p);
  }
  return cache[dev];
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Entry { const void* k; int dev; int bytes; };
  static std::mutex mu;
  static Entry seen[256];
  static int n_seen = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].k == kernel && seen[i].dev == dev && seen[i].bytes >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && n_seen < 256) seen[n_seen++] = Entry{kernel, dev, bytes};
  return e;
}

// setmaxnreg moves registers between the warps of a CTA, but only within what the CTA got at
// launch (registers per thread x threads); a role asking for more than its share of that pool
// would wait for ever.  Refuse to launch instead.
cudaError_t check_register_budget(const void* kernel, int threads, int regs_wanted_total) {
  struct Entry { const void* k; int total; };
  static std::mutex mu;
  static Entry seen[256];
  static int n_seen = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].k == kernel) return regs_wanted_total <= seen[i].total ? cudaSuccess : cudaErrorLaunchOutOfResources;
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
  if (e != cudaSuccess) return e;
  const int total = attr.numRegs * threads;
  if (n_seen < 256) seen[n_seen++] = Entry{kernel, total};
  return regs_wanted_total <= total ? cudaSuccess : cudaErrorLaunchOutOfResources;
}

namespace {

constexpr int kHeadDim = 128;

// Every entry point calls this after its host-side validation and before its first launch.  It
// also drops an error an earlier runtime call of this host thread may have left behind (the
// application's or this library's), so that the status read after a launch is that launch's own.
int check_arch() {
  static std::mutex mu;
  static int cached[64];
  static bool have[64] = {false};
  (void)cudaGetLastError();
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ASUKA_ERR_CUDA;
  if (dev < 0 || dev >= 64) return ASUKA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return ASUKA_ERR_CUDA;
    cached[dev] = major;
    have[dev] = true;
  }
  return cached[dev] == 10 ? ASUKA_OK : ASUKA_ERR_UNSUPPORTED_ARCH;
}

// multiprocessor count of the current device (the persistent kernels launch one CTA per SM)
int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
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

int make_map(CUtensorMap* m, const asuka_tensor& t, uint32_t box_rows = 128) {
  int r = tma_host::make_bshd_map(m, t.ptr, t.dtype == ASUKA_BF16, t.shape[0], t.shape[1], t.shape[2],
                                  t.shape[3], t.stride[0], t.stride[1], t.stride[2], box_rows);
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
  // grouped-query attention: the query heads are a whole multiple of the key/value heads
  if (k.shape[0] != q.shape[0] || k.shape[2] > q.shape[2] || q.shape[2] % k.shape[2] != 0)
    return ASUKA_ERR_BAD_SHAPE;
  if (causal && k.shape[1] < q.shape[1]) return ASUKA_ERR_BAD_SHAPE;
  // work items and grids are counted in 32-bit integers: (batch, head) units x 128-row tiles
  {
    const int64_t units = q.shape[0] * q.shape[2];
    const int64_t tiles = (std::max(q.shape[1], k.shape[1]) + 127) / 128;
    if (units * tiles > 0x3fffffff) return ASUKA_ERR_TOO_LARGE;
  }
  if (std::isnan(scale) || std::isinf(scale)) return ASUKA_ERR_BAD_ARGUMENT;
  o->dtype = q.dtype;
  o->s.B = static_cast<int>(q.shape[0]);
  o->s.Sq = static_cast<int>(q.shape[1]);
  o->s.H = static_cast<int>(q.shape[2]);
  o->s.group = static_cast<int>(q.shape[2] / k.shape[2]);
  o->s.Skv = static_cast<int>(k.shape[1]);
  o->s.causal = causal ? 1 : 0;
  o->s.softmax_scale = scale > 0.f ? scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
  o->s.softcap = 0.f;
  o->s.bf16 = q.dtype == ASUKA_BF16;
  return ASUKA_OK;
}

int map_cuda(cudaError_t e) { return e == cudaSuccess ? ASUKA_OK : ASUKA_ERR_CUDA; }

// 256-byte aligned start of the usable part of an optional scratch area, and its size
void* align_ws(void* ws, size_t bytes, size_t* usable) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(ws);
  const uintptr_t up = (a + 255u) & ~static_cast<uintptr_t>(255u);
  if (ws == nullptr || up - a >= bytes) {
    *usable = 0;
    return nullptr;
  }
  *usable = bytes - (up - a);
  return reinterpret_cast<void*>(up);
}

int attn_fwd_impl(const asuka_attn_params* p, float* lse_override, cudaStream_t stream, void* ws = nullptr,
                  size_t ws_bytes = 0) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  QKV c;
  int r;
  if ((r = check_qk(p->q, p->k, p->softmax_scale, p->causal, &c)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->v, c.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->out, c.dtype)) != ASUKA_OK) return r;
  for (int i = 0; i < 4; ++i) {
    if (p->v.shape[i] != p->k.shape[i] || p->out.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
  }
  if (std::isnan(p->softcap) || std::isinf(p->softcap) || p->softcap < 0.f) return ASUKA_ERR_BAD_ARGUMENT;
  c.s.softcap = p->softcap;
  float* lse = lse_override;
  if (lse == nullptr && p->lse.ptr != nullptr) {
    const int64_t shp[3] = {c.s.B, c.s.H, c.s.Sq};
    if ((r = check_dense(p->lse, ASUKA_F32, 3, shp)) != ASUKA_OK) return r;
    lse = static_cast<float*>(p->lse.ptr);
  }
  if ((r = check_arch()) != ASUKA_OK) return r;
  CUtensorMap mq, mk, mv;
  if ((r = make_map(&mq, p->q)) || (r = make_map(&mk, p->k)) || (r = make_map(&mv, p->v))) return r;
  const int sms = sm_count();
  if (sms <= 0) return ASUKA_ERR_CUDA;
  size_t usable = 0;
  void* split_ws = align_ws(ws != nullptr ? ws : p->workspace, ws != nullptr ? ws_bytes : p->workspace_bytes, &usable);
  const int parts = attn_fwd_parts(c.s, sms, usable);
  return map_cuda(launch_attn_fwd(mq, mk, mv, p->out.ptr, p->out.stride[0], p->out.stride[1],
                                  p->out.stride[2], lse, c.s, sms, split_ws, parts, stream));
}


int check_er(const asuka_tensor& er, const AttnShape& s) {
  if (er.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (er.dtype != ASUKA_F32) return ASUKA_ERR_BAD_DTYPE;
  if (er.ndim != 4) return ASUKA_ERR_BAD_SHAPE;
  if (er.shape[0] != s.B || er.shape[1] != s.H || er.shape[2] != s.Sq || er.shape[3] != s.Skv)
    return ASUKA_ERR_BAD_SHAPE;
  if (er.stride[3] != 1 || er.stride[0] < 0 || er.stride[1] < 0 || er.stride[2] < 0)
    return ASUKA_ERR_BAD_STRIDE;
  if ((reinterpret_cast<uintptr_t>(er.ptr) & 3u) != 0) return ASUKA_ERR_MISALIGNED;
  return ASUKA_OK;
}

// validates a score request and fills the launch arguments; `lse` is the row statistic to read
int prep_scores(const asuka_score_params* p, bool rowstat, QKV* c, ScoreArgs* a) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  int r;
  if ((r = check_qk(p->q, p->k, p->softmax_scale, p->causal, c)) != ASUKA_OK) return r;
  if (p->mode != ASUKA_SCORE_SUM && p->mode != ASUKA_SCORE_SUM_SQ && p->mode != ASUKA_SCORE_PERTURBED &&
      p->mode != ASUKA_SCORE_CORM)
    return ASUKA_ERR_BAD_ARGUMENT;
  const int64_t lshape[3] = {c->s.B, c->s.H, c->s.Sq};
  const int64_t sshape[3] = {c->s.B, c->s.H, c->s.Skv};
  if ((r = check_dense(p->lse, ASUKA_F32, 3, lshape)) != ASUKA_OK) return r;
  std::memset(a, 0, sizeof(*a));
  a->mode = p->mode;
  a->lse2 = static_cast<const float*>(p->lse.ptr);
  a->tau = 1.f;
  if (!rowstat) {
    if ((r = check_dense(p->score, p->mode == ASUKA_SCORE_CORM ? ASUKA_U8 : ASUKA_F32, 3, sshape)) != ASUKA_OK)
      return r;
    a->score = static_cast<float*>(p->score.ptr);
    if (p->mode == ASUKA_SCORE_CORM) {
      const asuka_tensor& m = p->corm_mask;
      if (m.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
      if (m.dtype != ASUKA_F32) return ASUKA_ERR_BAD_DTYPE;
      if (m.ndim != 2 || m.shape[0] != c->s.Sq || m.shape[1] != c->s.Skv) return ASUKA_ERR_BAD_SHAPE;
      if (m.stride[1] != 1 || m.stride[0] < 0) return ASUKA_ERR_BAD_STRIDE;
      a->exp_rand = static_cast<const float*>(m.ptr);  // read like the noise operand, shared by b and h
      a->er_stride_b = 0;
      a->er_stride_h = 0;
      a->er_stride_q = m.stride[0];
    }
    if (p->mode == ASUKA_SCORE_SUM_SQ) {
      if ((r = check_dense(p->score_sq, ASUKA_F32, 3, sshape)) != ASUKA_OK) return r;
      a->score_sq = static_cast<float*>(p->score_sq.ptr);
    }
  }
  if (p->mode == ASUKA_SCORE_PERTURBED) {
    if (!(p->tau > 0.f) || std::isinf(p->tau)) return ASUKA_ERR_BAD_ARGUMENT;
    a->tau = p->tau;
    a->seed = p->seed;
    a->unit_offset = p->seed_unit_offset;
    if (p->exp_rand.ptr != nullptr) {
      if ((r = check_er(p->exp_rand, c->s)) != ASUKA_OK) return r;
      a->exp_rand = static_cast<const float*>(p->exp_rand.ptr);
      a->er_stride_b = p->exp_rand.stride[0];
      a->er_stride_h = p->exp_rand.stride[1];
      a->er_stride_q = p->exp_rand.stride[2];
    } else {
      // seeded noise: the generator packs (q, kv) into one 32-bit word
      if (c->s.Sq > 65536 || c->s.Skv > 65536) return ASUKA_ERR_TOO_LARGE;
    }
  } else if (rowstat) {
    return ASUKA_ERR_BAD_ARGUMENT;
  }
  return check_arch();
}

// `chained`: the kernel ahead in the stream is one of this library's that writes neither q nor k
int col_scores_impl(const asuka_score_params* p, cudaStream_t stream, bool chained = false, void* ws = nullptr,
                    size_t ws_bytes = 0, PendingChunkSum* pending = nullptr) {
  QKV c;
  ScoreArgs a;
  int r = prep_scores(p, false, &c, &a);
  if (r != ASUKA_OK) return r;
  a.chained = chained ? 1 : 0;
  CUtensorMap mq, mk;
  if ((r = make_map(&mq, p->q)) || (r = make_map(&mk, p->k))) return r;
  const int sms = sm_count();
  if (sms <= 0) return ASUKA_ERR_CUDA;
  size_t usable = 0;
  void* split_ws = align_ws(ws != nullptr ? ws : p->workspace, ws != nullptr ? ws_bytes : p->workspace_bytes, &usable);
  const int chunks = col_scores_chunks(c.s, a.mode, sms, usable);
  return map_cuda(launch_col_scores(mq, mk, a, c.s, split_ws, chunks, stream, pending));
}

int kf_rowstat_impl(const asuka_score_params* p, cudaStream_t stream) {
  QKV c;
  ScoreArgs a;
  int r = prep_scores(p, true, &c, &a);
  if (r != ASUKA_OK) return r;
  CUtensorMap mq, mk;
  if ((r = make_map(&mq, p->q)) || (r = make_map(&mk, p->k))) return r;
  return map_cuda(launch_kf_rowstat(mq, mk, a, static_cast<float*>(p->lse.ptr), c.s, stream));
}

constexpr int kSelectMaxS32 = 32768;  // 4-byte keys in shared memory
constexpr int kSelectMaxS64 = 16384;  // 8-byte keys (RoCo)

int select_impl(const asuka_select_params* p, cudaStream_t stream, const PendingChunkSum* pending = nullptr) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->score.ptr == nullptr || p->idx.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->mode != ASUKA_SELECT_TOPK && p->mode != ASUKA_SELECT_TOPK_RECENT && p->mode != ASUKA_SELECT_ROCO)
    return ASUKA_ERR_BAD_ARGUMENT;
  if (p->score.ndim != 3) return ASUKA_ERR_BAD_SHAPE;
  const int64_t B = p->score.shape[0], H = p->score.shape[1], S = p->score.shape[2];
  if (B <= 0 || H <= 0 || S <= 0) return ASUKA_ERR_BAD_SHAPE;
  const int64_t sshape[3] = {B, H, S};
  int r;
  if ((r = check_dense(p->score, ASUKA_F32, 3, sshape)) != ASUKA_OK) return r;
  const bool roco = p->mode == ASUKA_SELECT_ROCO;
  if (S > (roco ? kSelectMaxS64 : kSelectMaxS32) || B * H > 0x7fffffff) return ASUKA_ERR_TOO_LARGE;
  const int recent = p->mode == ASUKA_SELECT_TOPK_RECENT ? p->recent : 0;
  if (recent < 0 || recent > S) return ASUKA_ERR_BAD_ARGUMENT;
  if (p->k_keep < 1 || p->k_keep > S - recent) return ASUKA_ERR_BAD_ARGUMENT;
  if (roco) {
    if ((r = check_dense(p->score_sq, ASUKA_F32, 3, sshape)) != ASUKA_OK) return r;
    if (p->q_len < 1 || (p->q_len > S && !p->all_rows)) return ASUKA_ERR_BAD_ARGUMENT;
    if (p->mean.ptr != nullptr && (r = check_dense(p->mean, ASUKA_F32, 3, sshape)) != ASUKA_OK) return r;
    if (p->std.ptr != nullptr && (r = check_dense(p->std, ASUKA_F32, 3, sshape)) != ASUKA_OK) return r;
  }
  const int64_t ishape[3] = {B, H, p->k_keep + recent};
  if ((r = check_dense(p->idx, ASUKA_I32, 3, ishape)) != ASUKA_OK) return r;
  if ((r = check_arch()) != ASUKA_OK) return r;
  SelectArgs a;
  a.score = static_cast<const float*>(p->score.ptr);
  a.score_sq = roco ? static_cast<const float*>(p->score_sq.ptr) : nullptr;
  a.idx = static_cast<int32_t*>(p->idx.ptr);
  a.rows = static_cast<int>(B * H);
  a.S = static_cast<int>(S);
  a.k_keep = p->k_keep;
  a.recent = recent;
  a.q_len = p->q_len;
  a.mode = p->mode;
  a.all_rows = roco && p->all_rows ? 1 : 0;
  a.mean = roco ? static_cast<float*>(p->mean.ptr) : nullptr;
  a.std = roco ? static_cast<float*>(p->std.ptr) : nullptr;
  a.part = pending != nullptr ? pending->part : nullptr;
  a.part_sq = pending != nullptr ? pending->part_sq : nullptr;
  a.n_chunks = pending != nullptr ? pending->n_chunks : 0;
  return map_cuda(launch_select(a, stream));
}

int prep_sima(const asuka_sima_params* p, SimaShape* sh) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (!is_16bit(p->q.dtype)) return p->q.ptr == nullptr ? ASUKA_ERR_NULL_POINTER : ASUKA_ERR_BAD_DTYPE;
  int r;
  if ((r = check_bshd(p->q, p->q.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->k, p->q.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->v, p->q.dtype)) != ASUKA_OK) return r;
  for (int i = 0; i < 4; ++i)
    if (p->k.shape[i] != p->q.shape[i] || p->v.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
  sh->B = static_cast<int>(p->q.shape[0]);
  sh->S = static_cast<int>(p->q.shape[1]);
  sh->H = static_cast<int>(p->q.shape[2]);
  sh->bf16 = p->q.dtype == ASUKA_BF16;
  sh->out_f32 = p->out.dtype == ASUKA_F32;
  sh->ea = false;
  if (static_cast<int64_t>(sh->B) * sh->H > (1 << 20)) return ASUKA_ERR_TOO_LARGE;
  return ASUKA_OK;
}

int sima_impl(const asuka_sima_params* p, void* ws, size_t ws_bytes, cudaStream_t stream, bool ea) {
  SimaShape sh;
  int r = prep_sima(p, &sh);
  if (r != ASUKA_OK) return r;
  sh.ea = ea;
  if (sh.out_f32) {
    const asuka_tensor& o = p->out;
    if (o.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
    if (o.ndim != 4) return ASUKA_ERR_BAD_SHAPE;
    for (int i = 0; i < 4; ++i)
      if (o.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
    if (o.stride[3] != 1) return ASUKA_ERR_BAD_STRIDE;
    for (int i = 0; i < 3; ++i)
      if (o.stride[i] <= 0 || (o.stride[i] % 4) != 0) return ASUKA_ERR_BAD_STRIDE;
    if ((reinterpret_cast<uintptr_t>(o.ptr) & 15u) != 0) return ASUKA_ERR_MISALIGNED;
  } else {
    if ((r = check_bshd(p->out, p->q.dtype)) != ASUKA_OK) return r;
    for (int i = 0; i < 4; ++i)
      if (p->out.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
  }
  if (ws == nullptr) return ASUKA_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return ASUKA_ERR_MISALIGNED;
  if (ws_bytes < sima_workspace_bytes(sh)) return ASUKA_ERR_WORKSPACE_TOO_SMALL;
  if ((r = check_arch()) != ASUKA_OK) return r;
  CUtensorMap mq, mk, mv, mo;
  if ((r = make_map(&mq, p->q)) || (r = make_map(&mk, p->k)) || (r = make_map(&mv, p->v))) return r;
  if (!sh.out_f32) {
    if ((r = make_map(&mo, p->out))) return r;
  } else {
    mo = mq;
  }
  const int sms = sm_count();
  if (sms <= 0) return ASUKA_ERR_CUDA;
  CUtensorMap m64[3];  // the same tensors in boxes of 64 rows, for the single-kernel path's first phase
  if ((r = make_map(&m64[0], p->q, 64)) || (r = make_map(&m64[1], p->k, 64)) || (r = make_map(&m64[2], p->v, 64))) return r;
  return map_cuda(launch_sima(mq, mk, mv, mo, p->out.ptr, p->out.stride[0], p->out.stride[1],
                              p->out.stride[2], ws, sh, m64, sms, stream));
}

// forward + column scores (+ selection) on one stream; the row statistic lives in `ws`
enum CaseKind { CASE_H2O, CASE_ROCO, CASE_KF };

size_t case_rowstat_bytes(const asuka_case_params* p) {
  const size_t n = static_cast<size_t>(p->q.shape[0]) * p->q.shape[2] * p->q.shape[1];
  return ((n * sizeof(float) + 255) / 256) * 256 * 2;  // unperturbed + perturbed row statistics
}
// grouped-query attention also parks the per-query-head scores [B, H, Skv] before the group mean
size_t case_ws_bytes(const asuka_case_params* p) {
  size_t bytes = case_rowstat_bytes(p);
  if (p->k.ndim == 4 && p->k.shape[2] > 0 && p->q.shape[2] > p->k.shape[2]) {
    const size_t n = static_cast<size_t>(p->q.shape[0]) * p->q.shape[2] * p->k.shape[1];
    bytes += ((n * sizeof(float) + 255) / 256) * 256;
  }
  return bytes;
}

// what the split of work items would like on top of case_ws_bytes on the current device
size_t case_split_bytes(const asuka_case_params* p, CaseKind kind) {
  if (p->k.ndim != 4 || p->q.ndim != 4) return 0;
  const int sms = sm_count();
  if (sms <= 0) return 0;
  AttnShape s;
  std::memset(&s, 0, sizeof(s));
  s.B = static_cast<int>(p->q.shape[0]);
  s.Sq = static_cast<int>(p->q.shape[1]);
  s.H = static_cast<int>(p->q.shape[2]);
  s.Skv = static_cast<int>(p->k.shape[1]);
  const int mode = kind == CASE_H2O ? ASUKA_SCORE_SUM : kind == CASE_ROCO ? ASUKA_SCORE_SUM_SQ : ASUKA_SCORE_PERTURBED;
  const size_t fwd = attn_fwd_split_bytes(s, attn_fwd_parts(s, sms, ~static_cast<size_t>(0)));
  const size_t col = col_scores_split_bytes(s, mode, col_scores_chunks(s, mode, sms, ~static_cast<size_t>(0)));
  return ((col + 255) / 256) * 256 + fwd + 256;
}

int case_impl(const asuka_case_params* p, CaseKind kind, void* ws, size_t ws_bytes,
              cudaStream_t stream) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->q.ptr == nullptr || p->q.ndim != 4) return p->q.ptr ? ASUKA_ERR_BAD_SHAPE : ASUKA_ERR_NULL_POINTER;
  for (int i = 0; i < 3; ++i)
    if (p->q.shape[i] <= 0) return ASUKA_ERR_BAD_SHAPE;
  if (ws == nullptr) return ASUKA_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(ws) & 15u) != 0) return ASUKA_ERR_MISALIGNED;
  if (ws_bytes < case_ws_bytes(p)) return ASUKA_ERR_WORKSPACE_TOO_SMALL;
  const int64_t B = p->q.shape[0], Sq = p->q.shape[1], H = p->q.shape[2];
  float* lse = static_cast<float*>(ws);
  float* lse_kf = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + case_rowstat_bytes(p) / 2);
  float* head_scores = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + case_rowstat_bytes(p));

  // validate everything before the first launch
  asuka_tensor lse_t;
  std::memset(&lse_t, 0, sizeof(lse_t));
  lse_t.ptr = lse;
  lse_t.dtype = ASUKA_F32;
  lse_t.ndim = 3;
  lse_t.shape[0] = B; lse_t.shape[1] = H; lse_t.shape[2] = Sq;
  lse_t.stride[0] = H * Sq; lse_t.stride[1] = Sq; lse_t.stride[2] = 1;

  asuka_attn_params fp;
  std::memset(&fp, 0, sizeof(fp));
  fp.q = p->q; fp.k = p->k; fp.v = p->v; fp.out = p->out;
  fp.lse = lse_t;
  fp.softmax_scale = p->softmax_scale;
  fp.causal = p->causal;

  asuka_score_params sp;
  std::memset(&sp, 0, sizeof(sp));
  sp.q = p->q; sp.k = p->k; sp.lse = lse_t; sp.score = p->score; sp.score_sq = p->score_sq;
  sp.exp_rand = p->exp_rand;
  sp.softmax_scale = p->softmax_scale;
  sp.tau = p->tau;
  sp.seed = p->seed;
  sp.seed_unit_offset = p->seed_unit_offset;
  sp.causal = p->causal;
  sp.mode = kind == CASE_H2O ? ASUKA_SCORE_SUM : kind == CASE_ROCO ? ASUKA_SCORE_SUM_SQ : ASUKA_SCORE_PERTURBED;
  if (kind == CASE_KF) sp.lse.ptr = lse_kf;

  asuka_select_params lp;
  std::memset(&lp, 0, sizeof(lp));
  const bool want_idx = p->idx.ptr != nullptr;
  if (want_idx) {
    lp.score = p->score; lp.score_sq = p->score_sq; lp.idx = p->idx;
    lp.k_keep = p->k_keep;
    lp.recent = p->recent;
    lp.q_len = static_cast<int32_t>(Sq);
    lp.all_rows = p->causal ? 0 : 1;
    if (kind == CASE_ROCO) { lp.mean = p->roco_mean; lp.std = p->roco_std; }
    lp.mode = kind == CASE_H2O ? ASUKA_SELECT_TOPK_RECENT : kind == CASE_ROCO ? ASUKA_SELECT_ROCO : ASUKA_SELECT_TOPK;
  }

  // grouped-query attention (H2O only; cases/attn_h2o.py:42-46): the column kernel writes one
  // score row per QUERY head into the workspace, the group mean lands in p->score [B, Hkv, Skv]
  const int64_t Hkv = p->k.ndim == 4 ? p->k.shape[2] : 0;
  const bool gqa = Hkv > 0 && H > Hkv;
  asuka_tensor head_score_t;
  std::memset(&head_score_t, 0, sizeof(head_score_t));
  if (gqa) {
    if (kind != CASE_H2O) return ASUKA_ERR_BAD_SHAPE;
    const int64_t Skv = p->k.shape[1];
    head_score_t.ptr = head_scores;
    head_score_t.dtype = ASUKA_F32;
    head_score_t.ndim = 3;
    head_score_t.shape[0] = B; head_score_t.shape[1] = H; head_score_t.shape[2] = Skv;
    head_score_t.stride[0] = H * Skv; head_score_t.stride[1] = Skv; head_score_t.stride[2] = 1;
    const int64_t gshape[3] = {B, Hkv, Skv};
    int r0 = check_dense(p->score, ASUKA_F32, 3, gshape);
    if (r0 != ASUKA_OK) return r0;
    sp.score = head_score_t;
  }

  // dry validation pass: the three impls validate before launching, so run their checks first
  {
    QKV c; ScoreArgs a;
    int r = prep_scores(&sp, false, &c, &a);
    if (r != ASUKA_OK) return r;
    if ((r = check_bshd(p->v, c.dtype)) != ASUKA_OK) return r;
    if ((r = check_bshd(p->out, c.dtype)) != ASUKA_OK) return r;
    for (int i = 0; i < 4; ++i)
      if (p->v.shape[i] != p->k.shape[i] || p->out.shape[i] != p->q.shape[i]) return ASUKA_ERR_BAD_SHAPE;
    if (want_idx) {
      const int64_t S = p->score.shape[2];
      const bool roco = kind == CASE_ROCO;
      const int recent = kind == CASE_H2O ? p->recent : 0;
      if (S > (roco ? kSelectMaxS64 : kSelectMaxS32)) return ASUKA_ERR_TOO_LARGE;
      if (recent < 0 || recent > S || p->k_keep < 1 || p->k_keep > S - recent) return ASUKA_ERR_BAD_ARGUMENT;
      const int64_t ishape[3] = {B, gqa ? Hkv : H, p->k_keep + recent};
      if ((r = check_dense(p->idx, ASUKA_I32, 3, ishape)) != ASUKA_OK) return r;
      if (roco) {
        const int64_t kshape[3] = {B, H, S};
        if (p->roco_mean.ptr != nullptr && (r = check_dense(p->roco_mean, ASUKA_F32, 3, kshape)) != ASUKA_OK) return r;
        if (p->roco_std.ptr != nullptr && (r = check_dense(p->roco_std, ASUKA_F32, 3, kshape)) != ASUKA_OK) return r;
      }
    }
    // the group mean runs one grid row per (batch, K/V head)
    if (gqa && B * Hkv > 65535) return ASUKA_ERR_TOO_LARGE;
  }

  // whatever the caller gave beyond the required part lets the kernels split their work items:
  // first the column pass's partial sums (small), then the forward kernel's partial outputs
  uint8_t* extra = static_cast<uint8_t*>(ws) + case_ws_bytes(p);
  size_t extra_bytes = ws_bytes - case_ws_bytes(p);
  void* col_ws = nullptr;
  size_t col_bytes = 0;
  {
    QKV c; ScoreArgs a;
    if (prep_scores(&sp, false, &c, &a) == ASUKA_OK) {
      const int sms = sm_count();
      size_t usable = 0;
      void* base = align_ws(extra, extra_bytes, &usable);
      if (sms > 0 && base != nullptr) {
        const size_t want = col_scores_split_bytes(c.s, a.mode, col_scores_chunks(c.s, a.mode, sms, usable));
        if (want > 0) {
          col_ws = base;
          col_bytes = want;
          const size_t step = ((want + 255) / 256) * 256;
          extra = static_cast<uint8_t*>(base) + step;
          extra_bytes = usable > step ? usable - step : 0;
        }
      }
    }
  }
  int r = attn_fwd_impl(&fp, nullptr, stream, extra_bytes > 0 ? extra : nullptr, extra_bytes);
  if (r != ASUKA_OK) return r;
  if (kind == CASE_KF) {
    if ((r = kf_rowstat_impl(&sp, stream)) != ASUKA_OK) return r;
  }
  // with a selection to follow (and no group mean in between) the selection kernel adds the column
  // pass's partial sums itself: one launch fewer
  PendingChunkSum pending;
  pending.n_chunks = 0;
  if ((r = col_scores_impl(&sp, stream, true, col_ws, col_bytes, want_idx && !gqa ? &pending : nullptr)) != ASUKA_OK)
    return r;
  if (gqa) {
    r = map_cuda(launch_group_mean(head_scores, static_cast<float*>(p->score.ptr), static_cast<int>(B * Hkv),
                                   static_cast<int>(H / Hkv), static_cast<int>(p->k.shape[1]), stream));
    if (r != ASUKA_OK) return r;
  }
  if (want_idx) r = select_impl(&lp, stream, pending.n_chunks > 0 ? &pending : nullptr);
  return r;
}

// ---- scratch for asuka_b200_h2o_static -------------------------------------------------------
// The array lives in the library's device image: one copy per GPU that loads the library.
// In HOST code the name `g_h2o_static_scratch` is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device
// with that device current.
constexpr size_t kStaticScratchBytes = static_cast<size_t>(ASUKA_H2O_STATIC_MAX_ROWS) * sizeof(float) * 2;
static __device__ __align__(256) unsigned char g_h2o_static_scratch[kStaticScratchBytes];

int h2o_static_scratch(void** out) {
  static std::mutex mu;
  static void* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ASUKA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_h2o_static_scratch);
    if (e != cudaSuccess || p == nullptr) return ASUKA_ERR_CUDA;
    cache[dev] = p;
  }
  *out = cache[dev];
  return ASUKA_OK;
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

int asuka_b200_selftest_wait_timeout(uint32_t limit_us, asuka_stream stream) {
  if (limit_us == 0 || limit_us > 100000) return ASUKA_ERR_BAD_ARGUMENT;
  const int r = check_arch();
  if (r != ASUKA_OK) return r;
  return map_cuda(launch_wait_selftest(static_cast<uint64_t>(limit_us) * 1000ull, static_cast<cudaStream_t>(stream)));
}

int asuka_b200_attn_fwd(const asuka_attn_params* p, asuka_stream stream) {
  return attn_fwd_impl(p, nullptr, static_cast<cudaStream_t>(stream));
}

int asuka_b200_col_scores(const asuka_score_params* p, asuka_stream stream) {
  return col_scores_impl(p, static_cast<cudaStream_t>(stream));
}

int asuka_b200_keyformer_rowstat(const asuka_score_params* p, asuka_stream stream) {
  return kf_rowstat_impl(p, static_cast<cudaStream_t>(stream));
}

int asuka_b200_select_topk(const asuka_select_params* p, asuka_stream stream) {
  return select_impl(p, static_cast<cudaStream_t>(stream));
}

int asuka_b200_pool_scores(const asuka_tensor* score, const asuka_tensor* out, int32_t kernel_size,
                           asuka_stream stream) {
  if (score == nullptr || out == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (score->ptr == nullptr || out->ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (score->ndim != 3) return ASUKA_ERR_BAD_SHAPE;
  const int64_t shp[3] = {score->shape[0], score->shape[1], score->shape[2]};
  for (int i = 0; i < 3; ++i)
    if (shp[i] <= 0) return ASUKA_ERR_BAD_SHAPE;
  int r;
  if ((r = check_dense(*score, ASUKA_F32, 3, shp)) != ASUKA_OK) return r;
  if ((r = check_dense(*out, ASUKA_F32, 3, shp)) != ASUKA_OK) return r;
  if (kernel_size < 1 || (kernel_size % 2) == 0 || kernel_size > 1025) return ASUKA_ERR_BAD_ARGUMENT;
  if (shp[0] * shp[1] > 65535 || shp[2] > (1 << 24)) return ASUKA_ERR_TOO_LARGE;
  if (out->ptr == score->ptr) return ASUKA_ERR_BAD_ARGUMENT;
  if ((r = check_arch()) != ASUKA_OK) return r;
  return map_cuda(launch_pool_scores(static_cast<const float*>(score->ptr), static_cast<float*>(out->ptr),
                                     static_cast<int>(shp[0] * shp[1]), static_cast<int>(shp[2]),
                                     kernel_size, static_cast<cudaStream_t>(stream)));
}

int asuka_b200_linattn32_fwd(const asuka_linattn32_params* p, asuka_stream stream) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  const asuka_tensor* ts[4] = {&p->q, &p->k, &p->v, &p->out};
  for (int i = 0; i < 4; ++i) {
    const asuka_tensor& t = *ts[i];
    if (t.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
    if (t.dtype != ASUKA_F32) return ASUKA_ERR_BAD_DTYPE;
    if (t.ndim != 4 || t.shape[3] != 32) return ASUKA_ERR_BAD_SHAPE;
    for (int d = 0; d < 4; ++d)
      if (t.shape[d] <= 0 || t.shape[d] != p->q.shape[d]) return ASUKA_ERR_BAD_SHAPE;
    if (t.stride[3] != 1) return ASUKA_ERR_BAD_STRIDE;
    for (int d = 0; d < 3; ++d)
      if (t.stride[d] <= 0 || (t.stride[d] % 4) != 0) return ASUKA_ERR_BAD_STRIDE;
    if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return ASUKA_ERR_MISALIGNED;
  }
  if (p->ea != 0 && p->ea != 1) return ASUKA_ERR_BAD_ARGUMENT;
  if (p->q.shape[0] * p->q.shape[2] > (1 << 24) || p->q.shape[1] > (1 << 24)) return ASUKA_ERR_TOO_LARGE;
  int r;
  if ((r = check_arch()) != ASUKA_OK) return r;
  LinAttn32Args a;
  a.q = static_cast<const float*>(p->q.ptr);
  a.k = static_cast<const float*>(p->k.ptr);
  a.v = static_cast<const float*>(p->v.ptr);
  a.out = static_cast<float*>(p->out.ptr);
  a.B = static_cast<int>(p->q.shape[0]); a.N = static_cast<int>(p->q.shape[1]); a.H = static_cast<int>(p->q.shape[2]);
  a.ea = p->ea;
  a.q_sb = p->q.stride[0]; a.q_sn = p->q.stride[1]; a.q_sh = p->q.stride[2];
  a.k_sb = p->k.stride[0]; a.k_sn = p->k.stride[1]; a.k_sh = p->k.stride[2];
  a.v_sb = p->v.stride[0]; a.v_sn = p->v.stride[1]; a.v_sh = p->v.stride[2];
  a.o_sb = p->out.stride[0]; a.o_sn = p->out.stride[1]; a.o_sh = p->out.stride[2];
  return map_cuda(launch_linattn32(a, static_cast<cudaStream_t>(stream)));
}

int asuka_b200_gather_kv(const asuka_gather_params* p, asuka_stream stream) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (!is_16bit(p->k.dtype)) return p->k.ptr == nullptr ? ASUKA_ERR_NULL_POINTER : ASUKA_ERR_BAD_DTYPE;
  int r;
  if ((r = check_bshd(p->k, p->k.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->v, p->k.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->k_out, p->k.dtype)) != ASUKA_OK) return r;
  if ((r = check_bshd(p->v_out, p->k.dtype)) != ASUKA_OK) return r;
  const int64_t B = p->k.shape[0], S = p->k.shape[1], H = p->k.shape[2];
  if (p->idx.ptr == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->idx.ndim != 3 || p->idx.shape[0] != B || p->idx.shape[1] != H || p->idx.shape[2] <= 0)
    return ASUKA_ERR_BAD_SHAPE;
  const int64_t n = p->idx.shape[2];
  const int64_t ishape[3] = {B, H, n};
  if ((r = check_dense(p->idx, ASUKA_I32, 3, ishape)) != ASUKA_OK) return r;
  for (int i = 0; i < 4; ++i) {
    if (p->v.shape[i] != p->k.shape[i] || p->v.stride[i] != p->k.stride[i]) return ASUKA_ERR_BAD_SHAPE;
    if (p->v_out.shape[i] != p->k_out.shape[i] || p->v_out.stride[i] != p->k_out.stride[i]) return ASUKA_ERR_BAD_SHAPE;
  }
  if (p->k_out.shape[0] != B || p->k_out.shape[1] != n || p->k_out.shape[2] != H) return ASUKA_ERR_BAD_SHAPE;
  if ((r = check_arch()) != ASUKA_OK) return r;
  GatherArgs a;
  a.k = static_cast<const uint16_t*>(p->k.ptr);
  a.v = static_cast<const uint16_t*>(p->v.ptr);
  a.k_out = static_cast<uint16_t*>(p->k_out.ptr);
  a.v_out = static_cast<uint16_t*>(p->v_out.ptr);
  a.idx = static_cast<const int32_t*>(p->idx.ptr);
  a.B = static_cast<int>(B); a.H = static_cast<int>(H); a.S = static_cast<int>(S); a.n = static_cast<int>(n);
  a.in_sb = p->k.stride[0]; a.in_ss = p->k.stride[1]; a.in_sh = p->k.stride[2];
  a.out_sb = p->k_out.stride[0]; a.out_ss = p->k_out.stride[1]; a.out_sh = p->k_out.stride[2];
  return map_cuda(launch_gather_kv(a, static_cast<cudaStream_t>(stream)));
}

int asuka_b200_sima_workspace_bytes(const asuka_sima_params* p, size_t* bytes) {
  if (bytes == nullptr) return ASUKA_ERR_NULL_POINTER;
  SimaShape sh;
  int r = prep_sima(p, &sh);
  if (r != ASUKA_OK) return r;
  *bytes = sima_workspace_bytes(sh);
  return ASUKA_OK;
}

int asuka_b200_sima_fwd(const asuka_sima_params* p, void* ws, size_t ws_bytes, asuka_stream stream) {
  return sima_impl(p, ws, ws_bytes, static_cast<cudaStream_t>(stream), false);
}

int asuka_b200_ea_fwd(const asuka_sima_params* p, void* ws, size_t ws_bytes, asuka_stream stream) {
  return sima_impl(p, ws, ws_bytes, static_cast<cudaStream_t>(stream), true);
}

int asuka_b200_case_workspace_bytes(const asuka_case_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->q.ndim != 4) return ASUKA_ERR_BAD_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (p->q.shape[i] <= 0) return ASUKA_ERR_BAD_SHAPE;
  *bytes = case_ws_bytes(p);
  return ASUKA_OK;
}

int asuka_b200_case_workspace_bytes_split(const asuka_case_params* p, size_t* bytes) {
  const int r = asuka_b200_case_workspace_bytes(p, bytes);
  // required part + what the work-item splits would like; RoCo's column pass asks most
  if (r == ASUKA_OK) *bytes += case_split_bytes(p, CASE_ROCO);
  return r;
}

int asuka_b200_attn_workspace_bytes(const asuka_attn_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr) return ASUKA_ERR_NULL_POINTER;
  QKV c;
  int r = check_qk(p->q, p->k, p->softmax_scale, p->causal, &c);
  if (r != ASUKA_OK) return r;
  const int sms = sm_count();
  if (sms <= 0) return ASUKA_ERR_CUDA;
  const size_t n = attn_fwd_split_bytes(c.s, attn_fwd_parts(c.s, sms, ~static_cast<size_t>(0)));
  *bytes = n > 0 ? n + 256 : 0;
  return ASUKA_OK;
}

int asuka_b200_col_scores_workspace_bytes(const asuka_score_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr) return ASUKA_ERR_NULL_POINTER;
  QKV c;
  int r = check_qk(p->q, p->k, p->softmax_scale, p->causal, &c);
  if (r != ASUKA_OK) return r;
  const int sms = sm_count();
  if (sms <= 0) return ASUKA_ERR_CUDA;
  const size_t n = col_scores_split_bytes(c.s, p->mode, col_scores_chunks(c.s, p->mode, sms, ~static_cast<size_t>(0)));
  *bytes = n > 0 ? n + 256 : 0;
  return ASUKA_OK;
}

int asuka_b200_h2o(const asuka_case_params* p, void* ws, size_t ws_bytes, asuka_stream stream) {
  return case_impl(p, CASE_H2O, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
// (the static array is handed over as exactly the required size: no work-item splitting here)
// H2O with the row statistic in the library's own fixed device array: no workspace argument, no
// allocation.  The size check comes first, so an oversized request never reaches a launch.  The
// first call on a device resolves the array's address (see h2o_static_scratch above).
int asuka_b200_h2o_static(const asuka_case_params* p, asuka_stream stream) {
  if (p == nullptr) return ASUKA_ERR_NULL_POINTER;
  if (p->q.ndim != 4) return ASUKA_ERR_BAD_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (p->q.shape[i] <= 0) return ASUKA_ERR_BAD_SHAPE;
  const double rows = static_cast<double>(p->q.shape[0]) * static_cast<double>(p->q.shape[1]) *
                      static_cast<double>(p->q.shape[2]);
  if (rows > static_cast<double>(ASUKA_H2O_STATIC_MAX_ROWS) || case_ws_bytes(p) > kStaticScratchBytes)
    return ASUKA_ERR_TOO_LARGE;
  int r = check_arch();  // (before the symbol lookup, which fails on a device the image was not built for)
  if (r != ASUKA_OK) return r;
  void* scratch = nullptr;
  r = h2o_static_scratch(&scratch);
  if (r != ASUKA_OK) return r;
  return case_impl(p, CASE_H2O, scratch, case_ws_bytes(p), static_cast<cudaStream_t>(stream));
}
int asuka_b200_roco(const asuka_case_params* p, void* ws, size_t ws_bytes, asuka_stream stream) {
  return case_impl(p, CASE_ROCO, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int asuka_b200_keyformer(const asuka_case_params* p, void* ws, size_t ws_bytes, asuka_stream stream) {
  return case_impl(p, CASE_KF, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
