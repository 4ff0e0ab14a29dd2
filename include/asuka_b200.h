/*
 * asuka_b200 -- C ABI of the hand-written sm_100a kernel library that stands in for the kernels
 * the FlashTensor/Asuka compiler generates for its fused-attention programs.
 *
 * What each entry point replaces in the reference:
 *   The reference emits, per fused kernel, a Python function
 *       def <KernelName>(arg0: torch.Tensor, ...) -> Tensor | Tuple[Tensor, ...]
 *   that allocates its outputs and launches one generated Triton kernel on the current stream
 *   (lib/Translate/to_triton.cpp:529-638).  The functions below are the bodies of those
 *   callables for the attention programs of cases/kernels/{attn,h2o,kf,roco}.py and
 *   bench/sima.mlir: plain pointers and sizes in, work enqueued on the given stream, integer
 *   status out.  The Python package `flashtensor_b200` wraps them back into the reference's
 *   per-case callables and its back-end plug-in interface (python/asuka/backend/builder.py:7-14).
 *
 * Conventions
 *   - Every function returns ASUKA_OK (0) or a negative asuka_status; nothing throws or aborts.
 *   - Arguments are validated on the host before anything is launched.
 *   - The library allocates nothing and keeps no pointer after a call returns.  The caller owns
 *     inputs, outputs and workspaces.
 *   - Work is enqueued on `stream` of the CURRENT device; calls do not synchronise.
 *   - Tensors are described by asuka_tensor: strides are in ELEMENTS; the innermost (head_dim)
 *     stride must be 1 and every other stride a multiple of 8 elements (16 bytes); base
 *     pointers must be 16-byte aligned.
 *   - q, k, v, out use the reference's [B, S, H, D] layout (cases/kernels/attn.py:37-39) with
 *     D = 128; the 2-D [S, H*D] layout of cases/attn.py is the same memory with B = 1.
 *   - Per-key scores use the reference's [B, H, S_kv] fp32 layout (cases/kernels/h2o.py:38).
 */
#ifndef ASUKA_B200_H_
#define ASUKA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  ASUKA_OK = 0,
  ASUKA_ERR_NULL_POINTER = -1,
  ASUKA_ERR_BAD_DTYPE = -2,
  ASUKA_ERR_BAD_SHAPE = -3,
  ASUKA_ERR_BAD_STRIDE = -4,
  ASUKA_ERR_MISALIGNED = -5,
  ASUKA_ERR_WORKSPACE_TOO_SMALL = -6,
  ASUKA_ERR_UNSUPPORTED_ARCH = -7,
  ASUKA_ERR_CUDA = -8,
  ASUKA_ERR_DEVICE_TIMEOUT = -9,
  ASUKA_ERR_BAD_ARGUMENT = -10,
  ASUKA_ERR_TOO_LARGE = -11
} asuka_status;

typedef enum { ASUKA_F16 = 0, ASUKA_BF16 = 1, ASUKA_F32 = 2, ASUKA_I32 = 3, ASUKA_U8 = 4 } asuka_dtype;

typedef struct {
  void* ptr;
  int32_t dtype; /* asuka_dtype */
  int32_t ndim;
  int64_t shape[5];
  int64_t stride[5]; /* in elements */
} asuka_tensor;

/* Opaque to C callers: a CUDA stream handle (cudaStream_t). */
typedef void* asuka_stream;

/* ---- attention forward: replaces the generated kernel for Attn.forward
 *      (cases/kernels/attn.py:18-34; unmasked form cases/attn.py:44-63). ---- */
typedef struct {
  asuka_tensor q;   /* [B, Sq,  H, 128] f16 | bf16 */
  asuka_tensor k;   /* [B, Skv, H, 128] same dtype */
  asuka_tensor v;   /* [B, Skv, H, 128] same dtype */
  asuka_tensor out; /* [B, Sq,  H, 128] same dtype */
  asuka_tensor lse; /* optional (ptr may be NULL): [B, H, Sq] f32, contiguous.  Receives the
                       base-2 log-sum-exp of the scaled logits of every query row; it is the
                       per-row statistic the column-score pass needs. */
  float softmax_scale; /* <= 0 selects 1/sqrt(128) */
  int32_t causal;      /* 1: key j is visible to query i iff j <= i + (Skv - Sq)
                          (torch.triu(-inf, diagonal=kv_len-q_len+1), cases/kernels/attn.py:22-23) */
  float softcap;       /* > 0: logits -> softcap * tanh(logits / softcap) before the mask, the
                          Gemma-2 variant (cases/kernels/gemma2.py:30-33); 0: off */
  void* workspace;     /* optional device scratch (256-byte aligned; may be NULL).  With few (batch,
                          head) units -- one GPU's share of a problem split over several -- the
                          kernel divides every work item's key range over several CTAs and parks
                          their partial results here; without it such launches leave SMs idle. */
  uint64_t workspace_bytes;
} asuka_attn_params;

int asuka_b200_attn_fwd(const asuka_attn_params* p, asuka_stream stream);
/* Scratch that lets asuka_b200_attn_fwd split key ranges on the current device for these shapes
 * (0 when the launch fills the device anyway).  Any smaller workspace is accepted too. */
int asuka_b200_attn_workspace_bytes(const asuka_attn_params* p, size_t* bytes);

/* ---- per-key column reductions of the attention probabilities: replaces the generated
 *      column kernel for h2o_score (cases/kernels/h2o.py:35-36), roco_score / roco_sq_score
 *      (cases/kernels/roco.py:42-46) and kf_score (cases/kernels/kf.py:36-40). ---- */
typedef enum {
  ASUKA_SCORE_SUM = 0,       /* sum_i p_ij                          (H2O)      */
  ASUKA_SCORE_SUM_SQ = 1,    /* sum_i p_ij and sum_i p_ij^2         (RoCo)     */
  ASUKA_SCORE_PERTURBED = 2, /* sum_i softmax_j((s_ij + g_ij)/tau)  (Keyformer) */
  ASUKA_SCORE_CORM = 3       /* any_i(p_ij >= mask_ij) -> 0/1 bytes  (CORM, cases/kernels/corm.py:34-37) */
} asuka_score_mode;

typedef struct {
  asuka_tensor q;        /* [B, Sq,  H, 128] */
  asuka_tensor k;        /* [B, Skv, H, 128] */
  asuka_tensor lse;      /* [B, H, Sq] f32: row statistic from asuka_b200_attn_fwd (modes 0, 1) or
                            from asuka_b200_keyformer_rowstat (mode 2) */
  asuka_tensor score;    /* [B, H, Skv] f32 out (mode ASUKA_SCORE_CORM: u8, 1 where the key is kept) */
  asuka_tensor score_sq; /* [B, H, Skv] f32 out, mode ASUKA_SCORE_SUM_SQ only */
  asuka_tensor exp_rand; /* mode 2: [B, H, Sq, Skv] f32 > 0, noise g = -log(exp_rand)
                            (cases/kernels/kf.py:36-37); ptr NULL selects the seeded generator */
  float softmax_scale;
  float tau;             /* mode 2 temperature (cases/kernels/kf.py:8) */
  uint64_t seed;         /* mode 2 with exp_rand.ptr == NULL */
  int32_t causal;
  int32_t mode;          /* asuka_score_mode */
  asuka_tensor corm_mask; /* mode ASUKA_SCORE_CORM: [Sq, Skv] f32 thresholds (1/(i+1) in the reference's
                             prepare, cases/kernels/corm.py:46-48), shared by every batch and head */
  void* workspace;        /* optional device scratch (256-byte aligned; may be NULL): with few (batch,
                             head) units the query rows are divided over several CTAs per key block,
                             whose partial sums are parked here and added in a fixed order */
  uint64_t workspace_bytes;
  uint32_t seed_unit_offset; /* seeded noise: the noise of unit (b, h) is keyed by seed_unit_offset +
                                b * H + h.  A caller that holds a slice of the (batch, head) units of
                                a larger problem passes the index of its first unit and gets the
                                noise the whole problem would have had; 0 otherwise */
} asuka_score_params;

int asuka_b200_col_scores(const asuka_score_params* p, asuka_stream stream);
/* Scratch that lets asuka_b200_col_scores split the query rows on the current device (0 when the
 * launch fills the device anyway).  Any smaller workspace is accepted too. */
int asuka_b200_col_scores_workspace_bytes(const asuka_score_params* p, size_t* bytes);

/* Row statistic of Keyformer's perturbed softmax (base-2 log-sum-exp of (s + g)/tau per query
 * row), the input `lse` of asuka_b200_col_scores in mode ASUKA_SCORE_PERTURBED.  Uses q, k,
 * exp_rand | seed, tau, softmax_scale, causal of `p` and writes p->lse. */
int asuka_b200_keyformer_rowstat(const asuka_score_params* p, asuka_stream stream);

/* ---- heavy-hitter selection.  The reference has no counterpart (it stops at the scores);
 *      the rules are the ones the benchmark configuration states. ---- */
typedef enum {
  ASUKA_SELECT_TOPK = 0,        /* k largest keys, ties -> lower index                       */
  ASUKA_SELECT_TOPK_RECENT = 1, /* k largest among [0, S-recent) plus the last `recent`      */
  ASUKA_SELECT_ROCO = 2         /* k largest mean = sum/n_j, ties -> larger std, lower index */
} asuka_select_mode;

typedef struct {
  asuka_tensor score;    /* [B, H, S] f32, values >= 0 */
  asuka_tensor score_sq; /* [B, H, S] f32, mode ROCO only */
  asuka_tensor idx;      /* [B, H, k_keep (+ recent)] i32 out, ascending */
  int32_t k_keep;
  int32_t recent; /* mode TOPK_RECENT */
  int32_t q_len;  /* mode ROCO: n_j = q_len - max(0, j - (S - q_len)), the number of query rows
                     that attend to key j under the causal mask */
  int32_t mode;   /* asuka_select_mode */
  int32_t all_rows; /* mode ROCO: 1 = the scores come from unmasked attention, every key is seen by
                       all q_len rows (n_j = q_len); 0 = causal count above */
  asuka_tensor mean; /* mode ROCO, optional (ptr may be NULL): [B, H, S] f32 out, sum_j / n_j */
  asuka_tensor std;  /* mode ROCO, optional: [B, H, S] f32 out, sqrt(max(sumsq_j / n_j - mean_j^2, 0)) */
} asuka_select_params;

int asuka_b200_select_topk(const asuka_select_params* p, asuka_stream stream);

/* ---- SnapKV's score smoothing: out = avg_pool1d(score, kernel_size, padding = kernel_size / 2,
 *      stride 1) along the key axis (cases/kernels/snapkv.py:35-38).  `score` and `out` are
 *      [B, H, S] f32, contiguous, and must not overlap; kernel_size is odd. ---- */
int asuka_b200_pool_scores(const asuka_tensor* score, const asuka_tensor* out, int32_t kernel_size,
                           asuka_stream stream);

/* ---- KV-cache compaction, the step after a selection: k_out[b, n, h, :] = k[b, idx[b, h, n], h, :]
 *      and the same for v.  The reference has no counterpart (it stops at the scores).
 *      k, v: [B, S, H, 128] 16-bit with identical strides; idx: [B, H, n] i32 with values in [0, S);
 *      k_out, v_out: [B, n, H, 128], same dtype, identical strides. ---- */
typedef struct {
  asuka_tensor k, v, idx, k_out, v_out;
} asuka_gather_params;
int asuka_b200_gather_kv(const asuka_gather_params* p, asuka_stream stream);

/* ---- SimA softmax-free attention: replaces the generated kernels for bench/sima.mlir:13-17
 *      (L1 normalisation as lib/Dialect/Asuka/Transforms/LowerComplexReduce.cpp:44-69). ---- */
typedef struct {
  asuka_tensor q;   /* [B, S, H, 128] f16 | bf16 */
  asuka_tensor k;
  asuka_tensor v;
  asuka_tensor out; /* [B, S, H, 128] same dtype, or f32 */
} asuka_sima_params;

/* Bytes of device workspace asuka_b200_sima_fwd needs for these shapes (pure host function). */
int asuka_b200_sima_workspace_bytes(const asuka_sima_params* p, size_t* bytes);
int asuka_b200_sima_fwd(const asuka_sima_params* p, void* workspace, size_t workspace_bytes,
                        asuka_stream stream);

/* ---- EA attention: replaces the generated kernels for bench/ea.mlir:13-17,
 *      out = softmax(q over the 128 features) . (softmax(k over the sequence)^T . v) per (batch,
 *      head).  Same tensors, same workspace size (asuka_b200_sima_workspace_bytes) and same
 *      three-kernel streaming structure as SimA, plus a column-maximum pass over k. ---- */
int asuka_b200_ea_fwd(const asuka_sima_params* p, void* workspace, size_t workspace_bytes,
                      asuka_stream stream);

/* ---- SimA / EA attention core at the reference's own benchmark shapes (bench/sima.mlir:13-17,
 *      bench/ea.mlir:13-17: 64 x 4 heads x 784 x 32, f32): head_dim 32, f32 in and out.  q, k, v
 *      may be strided views of the fused QKV projection's output (the asuka.split + reshape +
 *      transpose of lines 6-12 then cost nothing); out [B, N, H, 32] is what lines 15-16 reshape
 *      into the output projection's input.  HBM-bound: plain CUDA-core kernel, no workspace. ---- */
typedef struct {
  asuka_tensor q;   /* [B, N, H, 32] f32, unit stride along the last axis, others multiples of 4 */
  asuka_tensor k;
  asuka_tensor v;
  asuka_tensor out; /* [B, N, H, 32] f32 */
  int32_t ea;       /* 0: SimA (L1 normalisation over the sequence), 1: EA (softmax normalisations) */
} asuka_linattn32_params;
int asuka_b200_linattn32_fwd(const asuka_linattn32_params* p, asuka_stream stream);

/* ---- fused cases: forward + column scores (+ selection) enqueued back to back on one stream.
 *      `workspace` holds the row statistics between the kernels: two arrays of B*H*Sq floats
 *      (unperturbed and Keyformer's perturbed one), each rounded up to 256 bytes, plus, when k
 *      and v have fewer heads than q, B*H*Skv floats for the per-query-head scores ahead of the
 *      group mean.  asuka_b200_case_workspace_bytes gives that figure, which is required.
 *      asuka_b200_case_workspace_bytes_split adds, for launches with too few (batch, head) units
 *      to fill the current device, the scratch that lets the kernels split their work items
 *      further; a workspace between the two sizes is accepted and used as far as it goes. ---- */
typedef struct {
  asuka_tensor q, k, v, out;
  asuka_tensor score;    /* h2o_score | kf_score | roco_score, [B, H, Skv] f32 */
  asuka_tensor score_sq; /* RoCo only */
  asuka_tensor exp_rand; /* Keyformer only; ptr NULL selects the seeded generator */
  asuka_tensor idx;      /* optional (ptr may be NULL): kept indices, i32 */
  float softmax_scale;
  float tau;
  uint64_t seed;
  int32_t causal;
  int32_t k_keep;
  int32_t recent;
  asuka_tensor roco_mean; /* RoCo with idx only, optional: per-key mean of the probabilities over the */
  asuka_tensor roco_std;  /* rows that attend to the key, and their standard deviation; [B, H, Skv] f32 */
  uint32_t seed_unit_offset; /* Keyformer with seeded noise: as in asuka_score_params */
} asuka_case_params;

int asuka_b200_case_workspace_bytes(const asuka_case_params* p, size_t* bytes);
int asuka_b200_case_workspace_bytes_split(const asuka_case_params* p, size_t* bytes);
/* H2O.forward, cases/kernels/h2o.py:18-38 (+ selection) */
int asuka_b200_h2o(const asuka_case_params* p, void* workspace, size_t workspace_bytes,
                   asuka_stream stream);
/* RoCo.forward, cases/kernels/roco.py:18-48 (+ selection) */
int asuka_b200_roco(const asuka_case_params* p, void* workspace, size_t workspace_bytes,
                    asuka_stream stream);
/* KeyFormer.forward, cases/kernels/kf.py:19-42 (+ selection) */
int asuka_b200_keyformer(const asuka_case_params* p, void* workspace, size_t workspace_bytes,
                         asuka_stream stream);

/* ---- H2O for callers that can neither pass scratch memory nor let the library allocate.
 *      This entry point has no counterpart in the reference, whose generated callables allocate
 *      whatever they need with torch.empty.
 *
 * Who needs it: a plug-in hosted by an inference engine whose enqueue hook must not allocate; a
 * serving process whose own memory pool already holds the whole device, so that a cudaMalloc made
 * on its behalf simply fails; a latency-critical loop that cannot afford the device-wide
 * synchronisation an allocation brings.  For them this variant of asuka_b200_h2o keeps the one
 * piece of scratch the case needs -- the per-row softmax statistic handed from the forward kernel
 * to the column-score kernel -- in a fixed array that is part of the library's device image.
 * It calls no cudaMalloc, cudaFree or any allocating routine; inputs and outputs still come from
 * the caller exactly as for asuka_b200_h2o (same parameter block, `idx` optional).
 *
 * Limits and rules:
 *  - B * H * Sq must not exceed ASUKA_H2O_STATIC_MAX_ROWS; larger problems are refused with
 *    ASUKA_ERR_TOO_LARGE before anything is launched (use asuka_b200_h2o with a workspace).
 *  - With grouped-query inputs (k and v with fewer heads than q) the per-query-head scores are
 *    parked in the same array ahead of the group mean: 8 * B*H*Sq + 4 * B*H*Skv bytes (each part
 *    rounded up to 256) must fit in the array's 4 MiB, or the call is refused the same way.
 *  - The array (4 MiB) occupies memory on every GPU that loads the library, until the process exits.
 *  - The first call on each device looks up the array's device address (the device must be current,
 *    as for every call here) and remembers it.  Make that first call ahead of any stream capture.
 *  - All calls on a device share the one array.  Nothing in it has to start at zero -- the forward
 *    kernel rewrites every row it later reads -- but two calls whose kernels overlap on the GPU
 *    (different streams, or different host threads) race on it: keep calls on a device in order.
 */
#define ASUKA_H2O_STATIC_MAX_ROWS 524288
int asuka_b200_h2o_static(const asuka_case_params* p, asuka_stream stream);

/* ---- library services ---- */
int asuka_b200_version(void);
const char* asuka_b200_strerror(int status);
/* Kernels bound every wait; one that gives up records it in a device-side word.  This reads the
 * word (synchronising the current device) and clears it: 0 = no time-out since the last read. */
int asuka_b200_device_status(uint32_t* out);
/* Self-test of that path: launches one thread that waits `limit_us` microseconds (1 .. 100000)
 * on a barrier nothing completes, through the same bounded wait the pipeline kernels use.  The
 * kernel gives up, records the time-out and returns; the next asuka_b200_device_status then
 * reports ASUKA_ERR_DEVICE_TIMEOUT with count 1 and site 99, and the device stays usable. */
int asuka_b200_selftest_wait_timeout(uint32_t limit_us, asuka_stream stream);
/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t asuka_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ASUKA_B200_H_ */
