// Launch helpers for the encode kernels (encode_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "encode_core.h"

namespace gtok {

size_t merge_smem_bytes();
cudaError_t configure_kernels();     // once per device, before the first launch
int pretok_blocks_per_sm();
int merge_blocks_per_sm();
void launch_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s);
void launch_pretok(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_merge(const EncodeArgs& a, int blocks, cudaStream_t s);

}  // namespace gtok
