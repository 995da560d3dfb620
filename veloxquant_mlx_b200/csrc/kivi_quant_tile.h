// Internal interface of the tile quantize kernel (head_dim 128, group 32, f16/bf16).
#pragma once
#include "common.cuh"

namespace vq {
bool kivi_quant_tile_supported(const vq_kivi_quant_args &a);
int32_t kivi_quant_tile_launch(const vq_kivi_quant_args &a, cudaStream_t st);
}  // namespace vq
