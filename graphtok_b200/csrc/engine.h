// Host-side engine behind the libgtok C ABI: owns the vocabulary tables in device
// memory and, per capacity, a context with its workspaces, pinned staging
// buffers and the captured CUDA graph (memset -> [normalisation] -> [document mask] ->
// pretok -> words -> miss -> assemble).  Plays the role of the reference's TokenizerCtx
// (src/tokenizer.cuh:132-548, launch_graph_core at src/tokenizer.cu:4654-4773),
// with work proportional to the input length rather than to the capacity.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "vocab_host.h"

namespace gtok {

class Engine {
public:
    // Returns nullptr and a reason on failure (bad file, no usable GPU, ...).
    static Engine* create(const std::string& tokenizer_json, std::string& err);
    ~Engine();

    // Return codes follow the C ABI: >= 0 token count, -1 error, -2 output too small, -3 text
    // longer than cap_bytes (for a vocabulary that declares NFC: the normalised text, which the
    // graph produces itself from the raw bytes given here).
    // `text` is host memory.  When `out_on_device` the ids are copied device-to-device.
    int64_t encode(const uint8_t* text, uint32_t len, uint32_t cap_bytes, uint32_t* out, uint32_t max_out, bool out_on_device);
    // Documents are concatenated in `bytes`; `doc_off` has n_docs + 1 ascending offsets.
    // `out_on_device`: out_tokens and out_doc_tok are device pointers, filled by device-to-device copies.
    int64_t encode_batch(const uint8_t* bytes, const uint32_t* doc_off, uint32_t n_docs, uint32_t cap_bytes,
                         uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_tok, bool out_on_device = false);

    // ids -> the bytes they spell (host buffers).  Returns the byte count, -1 on error (an id outside
    // the vocabulary included), -2 when `max_out` is too small; `need` (optional) receives the byte
    // count in both cases, `kernel_ms` (optional) the CUDA-event time of the decode graph.
    int64_t decode(const uint32_t* ids, uint32_t n, uint8_t* out, uint64_t max_out, uint64_t* need, float* kernel_ms);

    // Measurement entry points (the reference's stage_input / launch_graph_sync,
    // src/tokenizer.cuh:252-279): stage once, then time graph replays alone.
    int stage(const uint8_t* bytes, uint32_t len, const uint32_t* doc_off, uint32_t n_docs, uint32_t cap_bytes);
    int64_t replay_staged(float* ms_out);                 // one replay; CUDA-event time of the graph
    int64_t read_staged(uint32_t* out, uint32_t max_out, uint32_t* out_doc_tok);
    // Same work as one replay, launched kernel by kernel with an event between them:
    // ms_out[0..3] = pretok, words, miss, assemble kernels, ms_out[4] = whole sequence,
    // ms_out[5] = what runs before pretok (normalisation kernel, document-bit kernels).
    int64_t profile_staged(float* ms_out);
    // Boundary bits of the staged input as left by the last replay: one bit per byte,
    // set where a pre-token starts; writes (len + 31) / 32 words.
    int64_t read_boundaries(uint32_t* out_words, uint32_t max_words);
    // Device-side table block for callers inside the library (no-allocation entry point).
    // Diagnostics (contexts created with GTOK_PHASE_CLOCKS set): cycles per kernel phase, summed over blocks.
    int read_phase_clocks(unsigned long long* out32, bool reset);
    // The block timeline of the last replay (4 kernels x 1280 blocks x 8 nanosecond stamps); cleared by the read.
    int read_timeline(unsigned long long* out, uint32_t max_words);
    // What the last replay of the staged input handed from kernel to kernel:
    //   out[0] pre-tokens (boundary bits), out[1] pre-tokens the whole-word table did not know and their
    //   bytes out[2] (2..64 bytes, merged by a thread each), out[3] pre-tokens longer than 64 bytes and
    //   their bytes out[4], out[5] ids the miss kernel wrote.  Counted on the host from the lists and bits
    //   in device memory; -1 when nothing is staged.
    int read_work_stats(uint64_t* out6);
    const struct DeviceTables* device_tables() const;
    int device_index() const;

    const HostVocab& vocab() const { return hv_; }
    uint32_t vocab_size() const { return hv_.vocab_size; }
    std::string last_error() const { return last_error_; }
    // Number of kernel launches one replay makes (for reporting).
    int launches_per_replay(bool batch) const { return (batch ? 5 : 4) + (hv_.nfc ? (batch ? 4 : 3) : 0); }
    void table_bytes(uint64_t* merge, uint64_t* word, uint64_t* other) const;

private:
    Engine() = default;
    struct Impl;
    std::unique_ptr<Impl> impl_;
    HostVocab hv_;
    std::string last_error_;
};

}  // namespace gtok
