/* libgtok C ABI: text -> token ids for byte-level BPE tokenizers on one B200.
 *
 * The first thirteen entry points are the reference's own C ABI
 * (src/gtok_shim.cc:133-399, exported through src/gtok.map:4-7) with the same
 * names, argument meaning and return codes, so that its ctypes / dlopen callers
 * (python/gpu_bpe_tokenizer/vllm.py:87-121, integrations/dynamo) bind unchanged.
 * The gtok_x_* entry points are additions for measurement and diagnostics.
 *
 * Ownership: the caller owns every input and output buffer; a handle owns its
 * device and pinned memory.  No exception crosses this boundary: failures are
 * negative return codes (or NULL).  A tokenizer handle is not thread-safe; a
 * dispatcher handle is.
 *
 * This library has no CPU route: gtok_cpu_backend() is always "off" (a state the
 * reference also has, src/cpu_route.cc:68-74) and every encode runs on the GPU;
 * creation fails when no sm_100 device is present.
 */
#ifndef GTOK_H
#define GTOK_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* src/gtok_shim.cc:138-155.  Loads an HF tokenizer.json; max_bytes is the largest
 * input a call may carry (raised to 4096).  GPU contexts are built on first use.
 * NULL on failure (see gtok_x_last_error). */
void* gtok_create(const char* vocab_json_path, uint32_t max_bytes);

/* src/gtok_shim.cc:160-202.  Returns the token count, -1 on error, -2 if `out` is too
 * small, -3 if the (normalised) input exceeds the handle's byte cap. */
int32_t gtok_encode(void* handle, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out);

/* src/gtok_shim.cc:209-236.  As gtok_encode, ids copied device-to-device into out_dev. */
int32_t gtok_encode_to_device(void* handle, const uint8_t* text, uint32_t len, void* out_dev, uint32_t max_out);

/* src/gtok_shim.cc:246-318.  n_docs documents concatenated in concat_bytes with
 * n_docs+1 byte offsets; one graph replay; result equals per-document gtok_encode
 * concatenated.  out_doc_offsets gets n_docs+1 running token counts.  Returns the
 * total, -1 error, -2 out_tokens too small, -3 bytes exceed the cap, -4 document
 * capacity could not grow. */
int32_t gtok_encode_batch(void* handle, const uint8_t* concat_bytes, const uint32_t* doc_byte_offsets, uint32_t n_docs,
                          uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_offsets);

/* src/gtok_shim.cc:325-335.  CPU-route controls; the route does not exist here:
 * the limit reads 0, setting it is accepted and ignored, the backend is "off". */
uint32_t gtok_cpu_max_bytes(void* handle);
void gtok_set_cpu_max_bytes(void* handle, uint32_t max_bytes);
const char* gtok_cpu_backend(void* handle);

/* src/gtok_shim.cc:346-390.  One dispatcher is shared by all request threads;
 * gtok_dispatch_encode is thread-safe and blocking.  policy: 0 adaptive, 1 GPU,
 * 2 CPU (accepted; every request still runs on the GPU).  Stats: [cpu_requests,
 * gpu_requests, gpu_batches, gpu_large, gpu_batch_ns]. */
void* gtok_dispatcher_create(const char* vocab_json_path, uint32_t cpu_workers, uint32_t max_batch_bytes,
                             uint32_t max_batch_docs, uint32_t policy);
int32_t gtok_dispatch_encode(void* dispatcher, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out);
void gtok_dispatcher_stats(void* dispatcher, uint64_t* out5);
void gtok_dispatcher_destroy(void* dispatcher);

/* src/gtok_shim.cc:392-399. */
uint32_t gtok_vocab_size(void* handle);
void gtok_destroy(void* handle);

/* ---- additions (no counterpart in the reference's C ABI) -------------------- */

/* Last failure message of this thread's most recent failing call ("" if none). */
const char* gtok_x_last_error(void);
/* 0 GPT-2, 1 Llama-3, 2 Qwen2.5; bit 8 set when the vocabulary asks for NFC. */
uint32_t gtok_x_family(void* handle);
/* Measurement, after the reference's stage_input / launch_graph_sync / read_staged_batch
 * (src/tokenizer.cuh:252-279): copy the input to the device once, then time graph
 * replays on their own.  doc_byte_offsets may be NULL for a single document.
 * gtok_x_replay returns the token count and writes the CUDA-event time of the replay. */
int32_t gtok_x_stage(void* handle, const uint8_t* bytes, uint32_t len, const uint32_t* doc_byte_offsets, uint32_t n_docs);
int32_t gtok_x_replay(void* handle, float* ms_out);
int32_t gtok_x_read(void* handle, uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_offsets);
/* Boundary bits of the staged input after a replay: bit i of the stream is set where a
 * pre-token starts at byte i.  Writes (len + 31) / 32 words; returns that count. */
int32_t gtok_x_read_boundaries(void* handle, uint32_t* out_words, uint32_t max_words);
/* The staged input once more, launched kernel by kernel with CUDA events between:
 * ms_out6 = {pre-tokenization, words, miss, assemble kernel, whole sequence, what runs before
 * pre-tokenization (normalisation and document-bit kernels)}. */
int32_t gtok_x_profile(void* handle, float* ms_out6);
/* Diagnostics: when the environment variable GTOK_PHASE_CLOCKS was set as the staged
 * context was created, SM cycles spent in each phase of the two kernels, summed over
 * thread blocks since the last reset (slots 0-6 pre-tokenization, 8-11 words, 12-15 assemble,
 * 16-20 miss, 24-26 normalisation).  -1 if off. */
int32_t gtok_x_phase_clocks(void* handle, uint64_t* out32, int32_t reset);
/* Diagnostics, same switch: when each thread block of the last replay's four kernels started,
 * finished, and finished its first six work items, as stamps of the GPU's nanosecond timer:
 * out[(kernel * 1280 + block) * 8 + slot], slot 0 = start, 1 = end, 2.. = work items; kernel 0
 * pre-tokenization, 1 words, 2 miss, 3 assemble.  Returns the words written (at most 40960),
 * -1 if off.  The record is cleared by the call. */
int32_t gtok_x_timeline(void* handle, uint64_t* out, uint32_t max_words);
/* gtok_encode_batch with the ids and the n_docs + 1 token offsets left in device memory (device-to-
 * device copies), as gtok_encode_to_device does for one document: what the reference's Python
 * Tokenizer.encode_batch_to_device returns (src/python_bindings.cc:410-507); its C ABI has no such entry. */
int32_t gtok_x_encode_batch_to_device(void* handle, const uint8_t* concat_bytes, const uint32_t* doc_byte_offsets, uint32_t n_docs,
                                      void* out_tokens_dev, uint32_t out_cap, void* out_doc_offsets_dev);
/* Raises the handle's byte cap (the limit behind return code -3) without re-creating the handle:
 * vocabulary and tables stay, the GPU context grows at the next call that needs it.  The reference
 * has callers re-create a bigger handle (src/gtok_shim.cc:160-202), which reloads the vocabulary.
 * Returns the cap now in force (never lowered). */
uint32_t gtok_x_set_max_bytes(void* handle, uint32_t max_bytes);
/* What the last replay of the staged input handed from kernel to kernel, for byte accounting:
 * out6 = {pre-tokens, pre-tokens of 2..64 bytes the whole-word table did not know, their bytes,
 * pre-tokens longer than 64 bytes, their bytes, ids written by the miss kernel}.  Counted on the
 * host from the lists and boundary bits in device memory (a debugging-speed call).  0 or -1. */
int32_t gtok_x_work_stats(void* handle, uint64_t* out6);
/* Sizes in bytes of the merge table, the whole-word table and the remaining tables. */
void gtok_x_table_bytes(void* handle, uint64_t* out3);
/* Kernel launches one graph replay performs (single document / batch). */
int32_t gtok_x_launches_per_replay(void* handle, int32_t batch);

/* Pre-token boundaries for callers that must not allocate.  No counterpart in the
 * reference.  Some hosts of this library cannot call cudaMalloc when they need an
 * answer: a serving process whose framework has claimed the whole device for its own
 * memory pool, or a plug-in that was handed a fixed set of buffers and nothing else.  For
 * them this entry point runs the pre-tokenization kernel with all of its working memory
 * taken from an array that is part of the library's device image (about 0.5 MB, held on
 * every GPU that loads the library until the process exits), and calls no cudaMalloc,
 * cudaFree or any other allocating routine.  That fixed array is also the limit: inputs
 * above 4 MiB (4,194,304 bytes) are refused with -3 and a message in gtok_x_last_error.
 *   text_dev      device pointer, 16-byte aligned, one document of `len` bytes; the
 *                 buffer must be readable up to `len` rounded up to 16
 *   out_bits_dev  device pointer to ((len + 4095) / 4096) * 128 uint32; bit i of the
 *                 stream is set where a pre-token starts at byte i (same bits as
 *                 gtok_x_read_boundaries)
 *   cuda_stream   a cudaStream_t (NULL = default stream); the work is queued on it and
 *                 the call waits for it (cudaStreamSynchronize) before it returns
 * The handle (created earlier, when allocation was still possible) supplies the
 * vocabulary tables; its device is made current for the call and the caller's current
 * device is put back before returning.  The first call on a device looks up the array's
 * device address: make that first call before any stream capture begins.  All calls share
 * the one array, which keeps the previous call's contents (the parts that must start at
 * zero are cleared on the stream each time): two calls that overlap on the GPU race, so
 * serialise them.  Returns 0; -1 on error, which includes error bits raised by the kernel
 * itself (a wait on an earlier tile that gave up, as overlapping calls can cause); -3 when
 * `len` exceeds the limit. */
int32_t gtok_x_boundaries_noalloc(void* handle, const void* text_dev, uint32_t len, void* out_bits_dev, void* cuda_stream);

/* Raw bytes of token `id` (the spelling the ids decode to); returns the length, -1 for an
 * id outside the vocabulary.  Nothing is written when `cap` is too small. */
int32_t gtok_x_token_bytes(void* handle, uint32_t id, uint8_t* out, uint32_t cap);

/* Decoding on the device: `n` token ids -> the bytes they spell, one pass (lengths, scan,
 * gather) in a captured graph of its own.  Replaces the reference's TokenizerCtx::decode
 * (src/tokenizer.cu:5499-5573, kernels :5225-5275) behind Tokenizer.decode / decode_bytes
 * (src/python_bindings.cc:558-600); the reference's C ABI has no decode entry.  Host buffers.
 * Returns the byte count; -1 on error (an id outside the vocabulary included); -2 when
 * `max_out` is too small (out = NULL with max_out = 0 asks for the size).  `need_out` (may be NULL)
 * receives the byte count in both cases,
 * `kernel_ms` (may be NULL) the CUDA-event time of the graph. */
int64_t gtok_x_decode(void* handle, const uint32_t* ids, uint32_t n, uint8_t* out, uint64_t max_out, uint64_t* need_out, float* kernel_ms);

/* Partitioning over the GPUs of one box (no counterpart in the reference, which is
 * single-GPU).  gtok_x_plan_chunks cuts one document into n_parts pieces at
 * positions where a pre-token starts whatever precedes it (letter | space letter),
 * so that the pieces' ids concatenate to the ids of the whole; out_offsets gets
 * n_parts+1 byte offsets.  gtok_x_plan_documents cuts a batch into n_parts
 * contiguous document ranges of about equal bytes; out_doc_index gets n_parts+1
 * document indices.  Each part is then encoded by one GPU with gtok_encode /
 * gtok_encode_batch; only the parts' token counts cross GPUs. */
int32_t gtok_x_plan_chunks(void* handle, const uint8_t* text, uint64_t len, uint32_t n_parts, uint64_t* out_offsets);
int32_t gtok_x_plan_documents(const uint32_t* doc_byte_offsets, uint32_t n_docs, uint32_t n_parts, uint32_t* out_doc_index);

#ifdef __cplusplus
}
#endif
#endif
