// Steps of a transformer block that sit between two of its projections and move as many bytes as
// a projection's output: HBM-bound row kernels, no allocation.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

// In place on the q and k thirds of a fused projection's output qkv (rows, 3 * heads * head_dim),
// 16-bit: per row and head, RMS norm over the head (fp32 mean of squares, `a * w * (1 / sqrt(ms + eps))`,
// flint/cpu/normalizations.cc:33-70 with its division as one reciprocal per head; weight (head_dim)
// 16-bit or null), narrowed to the 16-bit
// type as the norm's output is, then the rotation of even/odd pairs
// (left = even cos - odd sin, right = even sin + odd cos: waifu/src/krea2/dit.rs:260-275) in fp32
// with one rounding. Row r has position r % tokens; cos and sin are <float>(tokens, head_dim / 2).
// The v third is not touched. head_dim 64, 128 or 256; every operand 16-byte aligned.
cudaError_t qk_norm_rope(void *qkv, int is_bf16, int64_t rows, int heads, int head_dim, int tokens,
                         const void *q_weight, const void *k_weight, const float *cos, const float *sin, float eps,
                         cudaStream_t stream);

}  // namespace flsm100
