// Scaled dot product attention for sm_100a: one pass over the keys with the online softmax, both
// products on tcgen05 tensor cores with the scores, the probabilities (two-tile kernel) and the
// block's output in tensor memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

// What flint's fl_attention takes for the masks none and causal (flint/capi.h:118-133,532-544,
// flint/operators.h:255-272): q (batch, heads, q_len, head_dim), k and v (batch, kv_heads, kv_len,
// head_dim), out like q; heads a multiple of kv_heads. Every tensor's last dimension is contiguous;
// the other strides are in elements and need not be those of a contiguous tensor (a model hands in
// (batch, length, heads, head_dim) transposed). Query i sits at position p = i + kv_len - q_len and
// sees every key (mask 0), keys 0 .. p (1, causal), the keys of p's own block of `block_size` and of
// every block before it (2, block causal) or of p's own block alone (3, block diagonal).
struct AttentionArgs {
  const void *q, *k, *v;
  void *out;
  int is_bf16;  // else half
  int batch, heads, kv_heads, q_len, kv_len, head_dim;
  int64_t q_stride[3], k_stride[3], v_stride[3], out_stride[3];  // batch, head, position
  int mask_type;   // fl_mask_type_t
  int block_size;  // of the block masks, else 0
  void *v_transposed;   // scratch of attention_scratch_bytes(): v as (batch * kv_heads, head_dim, padded kv_len)
  uint32_t *status;     // device word: the kernel records a wait that gave up (never a hang)
  cudaStream_t stream;
};

// head_dim 64 or 128; bases 16-byte aligned and strides multiples of 8 elements (TMA reads the
// operands); the causal masks need kv_len >= q_len, the block diagonal one kv_len == q_len.
bool attention_supported(const AttentionArgs &a, const char **why);
size_t attention_scratch_bytes(int batch, int kv_heads, int kv_len, int head_dim);
// Which kernel a call runs on: two tiles of queries per CTA or one, and whether v is read as it
// lies (then no scratch is needed and the call is one launch) or through its transposition.
struct AttentionPlan {
  bool two_tiles;
  bool v_direct;
  int launches;
};
AttentionPlan attention_plan(const AttentionArgs &a);
// One launch where two tiles of queries share a CTA (more than 128 queries, any mask but the block
// diagonal one, a v without repeated dimensions): v is read as it lies. Otherwise two: the
// transposition of v into the scratch, and the one-tile kernel.
cudaError_t attention(const AttentionArgs &a, const char **why);

constexpr uint32_t kStatusAttentionTimeout = 0x41;
constexpr uint32_t kStatusAttentionLayout = 0x42;  // dynamic shared memory did not start on a 1024-byte boundary

}  // namespace flsm100
