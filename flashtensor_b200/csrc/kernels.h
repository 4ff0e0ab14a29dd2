// Internal launch interface between the C-ABI layer (capi.cu) and the kernel files.
// All arguments have been validated by the caller.  Each function enqueues on `stream` and
// returns the launch's own cudaError_t (cudaGetLastError right after the launch), never synchronising.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

namespace asuka {

// Device-side record of bounded waits that expired: word 0 = count, word 1 = last site id.
uint32_t* device_status_words();  // device address of a 4-word __device__ array
void count_launch();
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of per call
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes);
// error unless the registers the kernel's roles ask for after setmaxnreg fit in what the CTA gets at launch
cudaError_t check_register_budget(const void* kernel, int threads, int regs_wanted_total);

// Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while
// the one ahead of it in the stream drains; it orders itself with griddepcontrol.wait.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

struct AttnShape {
  int B, H, Sq, Skv;  // H: query heads
  int group;          // query heads per key/value head (1: multi-head attention)
  int causal;
  float softmax_scale;
  float softcap;  // > 0: logits -> softcap * tanh(logits / softcap) before the mask; 0: off
  bool bf16;
};

// q/k/v tensor maps: [B,S,H,128] boxes of 64 x 1 x 128 x 1, 128-byte swizzle.  `out` is written
// with plain 16-byte stores (strides in elements).  `num_sms` sizes the persistent grid.
// `split_ws` / `parts`: optional key-range split (see attn_fwd_parts); parts = 1 or a null
// workspace runs every work item over its whole key range.
cudaError_t launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                            void* out, int64_t o_sb, int64_t o_ss, int64_t o_sh, float* lse2,
                            const AttnShape& s, int num_sms, void* split_ws, int parts, cudaStream_t stream);
// parts the key range is worth cutting into on `num_sms` SMs, limited by the workspace on offer
int attn_fwd_parts(const AttnShape& s, int num_sms, size_t ws_bytes);
size_t attn_fwd_split_bytes(const AttnShape& s, int parts);

struct ScoreArgs {
  const float* lse2;       // [B,H,Sq]
  float* score;            // [B,H,Skv]
  float* score_sq;         // [B,H,Skv] or null
  const float* exp_rand;   // [B,H,Sq,Skv] or null
  int64_t er_stride_b, er_stride_h, er_stride_q;  // elements (innermost stride 1)
  float tau;
  uint64_t seed;
  uint32_t unit_offset;    // seeded noise: index of this call's first (batch, head) unit in the whole problem
  int mode;                // asuka_score_mode
  int chained;             // 1: the kernel ahead in the stream is this library's own and writes none of
                           // q and k, so the K tiles may be fetched before that kernel has finished
};
// `split_ws` / `chunks`: optional query-range split (see col_scores_chunks); chunks = 1 or a null
// workspace gives every key block one CTA that walks all query tiles.
// `pending`: when non-null and the query-range split is active, the final sum of the partial
// results is left to the caller (the selection kernel can do it on its way in) and described here.
struct PendingChunkSum {
  const float* part;     // [n_chunks][rows * S]
  const float* part_sq;  // or null
  int n_chunks;          // 0: nothing pending, the scores are final
};
cudaError_t launch_col_scores(const CUtensorMap& mq, const CUtensorMap& mk, const ScoreArgs& a,
                              const AttnShape& s, void* split_ws, int chunks, cudaStream_t stream,
                              PendingChunkSum* pending = nullptr);
int col_scores_chunks(const AttnShape& s, int mode, int num_sms, size_t ws_bytes);
size_t col_scores_split_bytes(const AttnShape& s, int mode, int chunks);
// Keyformer row statistic: writes lse2' [B,H,Sq] of (s + g) / tau
cudaError_t launch_kf_rowstat(const CUtensorMap& mq, const CUtensorMap& mk, const ScoreArgs& a,
                              float* lse2_out, const AttnShape& s, cudaStream_t stream);

struct SelectArgs {
  const float* score;     // [B*H, S] rows, contiguous
  const float* score_sq;  // or null
  int32_t* idx;           // [B*H, n_out]
  int rows, S, k_keep, recent, q_len, mode;
  int all_rows;           // RoCo: every key is seen by all q_len rows (unmasked attention)
  // partial sums of a query-range split still to be added (in range order) into score / score_sq,
  // which the kernel then also writes; n_chunks = 0: the scores are final
  const float* part;
  const float* part_sq;
  int n_chunks;
  float* mean;            // RoCo, optional outputs [B*H, S]
  float* std;
};
cudaError_t launch_select(const SelectArgs& a, cudaStream_t stream);

// one thread waits `limit_ns` on a barrier nobody completes and records the time-out
cudaError_t launch_wait_selftest(uint64_t limit_ns, cudaStream_t stream);
// mean over each group of `group` consecutive heads: [rows * group, S] -> [rows, S]
cudaError_t launch_group_mean(const float* in, float* out, int rows, int group, int S, cudaStream_t stream);
// moving average over the key axis of [rows, S] scores (odd kernel size, zero padding)
cudaError_t launch_pool_scores(const float* in, float* out, int rows, int S, int ksize,
                               cudaStream_t stream);

// KV-cache compaction: rows of k and v (16-bit, [B,S,H,128], strides in elements, same for both)
// gathered at idx [B,H,n] into [B,n,H,128] outputs
struct GatherArgs {
  const uint16_t* k;
  const uint16_t* v;
  uint16_t* k_out;
  uint16_t* v_out;
  const int32_t* idx;
  int B, H, S, n;
  int64_t in_sb, in_ss, in_sh, out_sb, out_ss, out_sh;
};
cudaError_t launch_gather_kv(const GatherArgs& a, cudaStream_t stream);

// linear attention at head_dim 32, f32: q, k, v, out [B, N, H, 32], strides in elements (unit stride
// along the features, the others multiples of 4)
struct LinAttn32Args {
  const float* q;
  const float* k;
  const float* v;
  float* out;
  int B, N, H;
  int ea;  // 1: EA (softmax normalisations), 0: SimA (L1 normalisations)
  int64_t q_sb, q_sn, q_sh, k_sb, k_sn, k_sh, v_sb, v_sn, v_sh, o_sb, o_sn, o_sh;
};
cudaError_t launch_linattn32(const LinAttn32Args& a, cudaStream_t stream);

struct SimaShape {
  int B, H, S;
  bool bf16;
  bool out_f32;
  bool ea;  // the EA program (softmax normalisations) instead of SimA (L1 normalisations)
};
size_t sima_workspace_bytes(const SimaShape& s);
cudaError_t launch_sima(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mo, void* out_ptr, int64_t out_stride_b,
                        int64_t out_stride_s, int64_t out_stride_h, void* ws, const SimaShape& s,
                        const CUtensorMap* maps64, int num_sms, cudaStream_t stream);  // maps64: q, k, v with 64-row boxes

}  // namespace asuka
