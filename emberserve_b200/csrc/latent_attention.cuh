// Interface of the tensor-core latent attention kernel (latent_attention_mma.cu) towards the
// dispatcher in latent_attention.cu.  Arguments as for ems_latent_attention; bfloat16 only.
#pragma once

#include "common.cuh"

namespace ems {

// Whether the tensor-core kernel takes the geometry: a latent of a multiple of 32 numbers (up to
// 512), a rotated part of a multiple of 16, cached vectors on 16-byte boundaries.
bool latent_mma_supported(int R, int P, const void* qlat, const void* qrot, int q_row_stride, int q_head_stride,
                          const void* pages);

// `partial` ([token, head, split, R + 2] float: unnormalised sums, maximum in natural-log units,
// sum) is written instead of `out` when splits > 1; the caller runs the merge kernel.
int run_latent_mma(const void* qlat, const void* qrot, int q_row_stride, int q_head_stride, const void* pages,
                   const int* block_tables, int bt_stride, int page_size, const int* positions,
                   const int* row_of_token, void* out, float* partial, int num_tokens, int H, int R, int P,
                   float scale, int splits, cudaStream_t stream);

}  // namespace ems
