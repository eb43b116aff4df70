// The per-rank context behind the C-ABI handle: weights, caller-owned KV cache, private activations and scratch,
// captured CUDA graphs, the tensor-parallel communicator.  Shared by the translation units that string kernels into a
// step (api.cu: the Llama / Qwen2 decoder stack; stack.cu: models described layer by layer).
#pragma once
#include <nccl.h>  // types only; the library is resolved at run time from the process (torch's copy)
#include <string.h>

#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200 { struct StackModel; }

struct LayerW {
  const __nv_bfloat16 *ln1 = nullptr, *qkv = nullptr, *qkv_b = nullptr, *o = nullptr, *ln2 = nullptr, *gu = nullptr,
                      *down = nullptr;
  bool gu_interleaved = false;  // gu holds 128-row slabs of 64 gate rows + the 64 matching up rows
};

struct GraphKey {
  uint64_t parts[16];   // every pointer and size the captured graph baked in
  bool operator==(const GraphKey& o) const { return memcmp(parts, o.parts, sizeof(parts)) == 0; }
};
struct GraphKeyHash {
  size_t operator()(const GraphKey& k) const {
    uint64_t h = 0x1234;
    for (uint64_t v : k.parts) h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return (size_t)h;
  }
};

struct b200_ctx {
  b200_model_cfg cfg;
  int hq, hkv, inter, vocab_local, qkv_w;  // local (per TP rank) sizes
  int max_logit_rows;
  std::vector<LayerW> layers;
  const __nv_bfloat16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr, *cos_sin = nullptr;
  int64_t max_pos = 0;
  __nv_bfloat16 *kc = nullptr, *vc = nullptr;
  int64_t n_blocks = 0;
  // private device buffers
  void* pool = nullptr;
  int64_t pool_bytes = 0;
  __nv_bfloat16 *x, *res, *normed, *qkv_buf, *attn_out, *gu_buf, *act, *lm_in, *logits;
  float *sres, *ssq;   // fp32 residual stream [T][h] and its per-slab sums of squares [T][h/128] (norm folded into the linears)
  void* attn_ws;
  int64_t attn_ws_bytes;
  void* lin_ws;
  int64_t lin_ws_bytes;
  int32_t* d_meta;
  int64_t meta_ints;
  int32_t* d_tokens;
  float* d_max;
  float* d_pairs;     // [rows][2] local (max, idx)
  float* d_gathered;  // [world][rows][2]
  void* d_sample;     // sampling parameters of the rows, packed (b200_ctx_sample_last)
  void* d_logprob;    // [rows] chosen ids | [rows] logprob | [rows][32] top ids | [rows][32] top logprobs
  void* d_adjust;     // packed penalties / logit_bias of the step's rows (b200_ctx_adjust_last)
  int logits_ld = 0;           // leading dimension of `logits` (vocab_local, rounded up to 8 for layer-list models)
  float* logits_f32 = nullptr; // layer-list models in fp32 mode: the unrounded logit rows [rows][logits_ld]
  __nv_bfloat16* logits_full;  // TP only: [world][rows][vocab_local], gathered for the sampler
  // graphs
  bool graphs = true;
  std::unordered_map<GraphKey, cudaGraphExec_t, GraphKeyHash> graph_cache;
  int last_launches = 0;
  // taps
  int tap_layer = -1;
  void *tap_hidden = nullptr, *tap_res = nullptr;
  // TP
  ncclComm_t comm = nullptr;
  // all-reduce over peer memory (allreduce.cu): one IPC-shareable allocation per rank
  //   [ partial 0 | partial 1 | gather 0 | gather 1 | flag block (2 x 2 x 8 x 128 B) | state (counter[2], ticket[2]) ]
  char* ar_mem = nullptr;
  int64_t ar_buf_bytes = 0, ar_total_bytes = 0;
  char* ar_peer[8] = {};
  bool ar_ready = false;
  // a model described layer by layer (b200_stack_create): its own weights, caches and step; null for the fixed decoder stack
  b200::StackModel* stack = nullptr;
  int gemv_max_t = 0;  // rows <= this use the CUDA-core GEMV; 0: the tcgen05 path serves every T (measured faster)
  bool pdl = true;
  bool fuse = true;                    // epilogue fusion (RoPE+KV, SiLU*mul) on the tcgen05 path
  // Steps of at most this many rows fold the RMSNorms into the linears (0: off).  Measured on 8B: batch 1 3.05 -> 3.00
  // ms/step; at 64 rows every CTA of a consumer re-normalises 1 MiB of fp32 rows out of L2 and the step slows from 4.6
  // to 6.3 ms, so the fold stops at the 16-row tile.
  int fuse_norm_max_t = 16;
};


// One scheduler step as the C-ABI entry points hand it to the model's enqueue function.
struct StepArgs {
  const int32_t *ids, *positions, *slots, *block_table, *row_to_seq, *ctx_lens, *logit_rows;
  int bt_stride, T, max_ctx, R;
  int32_t* out_tokens;
  void* out_logits;
  int n_seqs = 0;   // sequences in the step when the caller knows it (host-buffer entry), else 0
  // host-buffer entry: the tokens the previous step left in the ctx; an id -(j+1) means "row j of those"
  const int32_t* prev_tokens = nullptr;
  int n_prev = 0;
  // models with per-sequence state: the state slot of each of the step's n_seqs sequences (host-buffer entry)
  const int32_t* seq_slots = nullptr;
};

namespace b200 {
// stack.cu: the step and readiness check of a layer-list model, and its teardown
int stack_enqueue_step(b200_ctx* c, const StepArgs& a, cudaStream_t s);
int stack_ready(const b200_ctx* c);
int stack_state_slots(const b200_ctx* c);
void stack_step_slots(const b200_ctx* c, const int32_t** seq_slots, int* n_seqs);   // what b200_stack_set_step_slots left   // > 0: the host-buffer step carries seq_slots behind its block tables
void stack_destroy(b200_ctx* c);
}  // namespace b200
