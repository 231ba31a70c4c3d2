// Launch helpers for the encode kernels (encode_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <string>

#include "decode_core.h"
#include "encode_core.h"

namespace gtok {

cudaError_t configure_kernels();     // once per device, before the first launch
int pretok_blocks_per_sm();
int words_blocks_per_sm();
int miss_blocks_per_sm();
int assemble_blocks_per_sm();
int nfc_blocks_per_sm();
int decode_blocks_per_sm();
void launch_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s);
void launch_raw_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s);   // over raw_doc_off
// check: the context's arguments with raw_docmask unset; copy and nfc: the context's own arguments
void launch_nfc_check(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_nfc_copy(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_nfc(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_pretok(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_words(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_miss(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_assemble(const EncodeArgs& a, int blocks, cudaStream_t s);
void launch_decode(const DecodeArgs& a, int blocks, cudaStream_t s);
// Addresses of two kernels as graph kernel nodes report them (to recognise the nodes that get an L2 access-policy window).
const void* words_kernel_address();
const void* miss_kernel_address();

// The single-block kernel for short single documents (tiny_kernel.cu): text of up to kTinyMaxBytes
// and {byte count, 1} in page-locked host memory the device can read; a.out_tokens and a.status may
// be page-locked host memory as well.  a.text, a.meta and the work buffers are device memory as ever.
constexpr uint32_t kTinyMaxBytes = 2048;
cudaError_t configure_tiny_kernel();
void launch_tiny(const EncodeArgs& a, const uint8_t* host_text, const uint32_t* host_meta, cudaStream_t s);


// Largest input of boundaries_noalloc(), fixed by its statically reserved working memory.
constexpr uint32_t kNoAllocMaxBytes = 4u << 20;
constexpr uint32_t kNoAllocTiles = kNoAllocMaxBytes / kTile;
// Boundary bits of `len` bytes of single-document text already in device memory, written
// to a caller-supplied device buffer, using only working memory reserved inside the
// library image.  See gtok_x_boundaries_noalloc in include/gtok.h for the contract.
int boundaries_noalloc(const DeviceTables& tb, int device, const void* text_dev, uint32_t len, void* out_bits_dev,
                       cudaStream_t stream, std::string& err);

}  // namespace gtok
