// Types shared by the paged decode attention kernels and their launchers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

constexpr int kMaxAttentionSplits = 64;
constexpr float kLog2e = 1.4426950408889634f;

// Kernel arguments of one paged decode attention launch. Split partials live in
// a caller-provided fp32 workspace: ws_ml[b][h][s] = (row max in the log2
// domain, softmax denominator), ws_acc[b][h][s][d] = unnormalised output.
struct AttnParams {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const void* kv_scales;   // 8-bit pools only: fp16 [slots][kv_heads][2 (K, V)][page_size], one scale per cached row
  int kv8;                 // the pools hold unsigned bytes: value = (byte - 128) * scale of its row
  int num_slots;           // slots of the pool (0: unknown); bounds the tensor maps of the fast kernels
  // Fused activation pre-pass of the projection that follows (null: off): the [batch][heads*head_dim] output also
  // leaves as the integer GEMM's fixed-point planes, scales and sums, rows batch..quant_rows-1 zeroed.
  int8_t* quant_planes;
  float* quant_sx;
  int* quant_qsum;
  int quant_rows;          // padded row count of the planes (16, 32 or 64)
  const int32_t* page_table;
  const int32_t* seq_lens;
  void* out;
  float* ws_ml;
  float* ws_acc;
  int batch, heads, kv_heads, max_pages, page_size, head_dim;
  int group;         // heads / kv_heads
  int head_chunks;   // CTAs along the query heads of one KV head
  int splits, chunk_tokens;
  long long q_stride, out_stride;  // elements between consecutive sequences
  float scale_log2;                // softmax_scale * log2(e)
};

// Resolve the number of context splits (requested == 0: choose) and the number
// of tokens each split covers (a multiple of page_size).
void resolve_attention_splits(int batch, int heads, int kv_heads, int max_pages, int page_size,
                              int requested, int* splits, int* chunk_tokens);

// Tensor-core path (fp16/bf16, head_dim 64/128, 16-token pages, GQA group <= 16).
// (8-bit pools: fp16 queries, head_dim 128.)
bool paged_attention_fast_supported(const AttnParams& p, int dtype);
int launch_paged_attention_fast(const AttnParams& p, int dtype, cudaStream_t stream);
// Can the fast kernel also write the fixed-point planes (single split, fp16 pages and queries, head_dim 128,
// the kv heads of a sequence as one thread-block cluster)?
bool paged_attention_quantize_supported(const AttnParams& p, int dtype);
int paged_attention_device_status(bool reset);

}  // namespace cb200
