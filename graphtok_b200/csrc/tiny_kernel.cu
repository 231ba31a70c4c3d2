// The whole encode path for a short input in ONE thread block: pre-tokenization, whole-word
// look-ups, merge loops and output assembly run one after the other in the same kernel, on the same
// tile programs as the four-kernel graph (encode_core.h), so that a prompt of a few kilobytes costs
// one kernel launch instead of a control-block reset and four launches with their gaps.  Plays the
// role of the reference's single-CTA front end and tail (src/tokenizer.cu:3259-3396, :3416-3463).
//
// The kernel reads what it wrote itself (boundary bits, slots, lists), so every load of such data
// must be an ordinary one: GTOK_COHERENT_LOADS turns the non-coherent loads of encode_core.h off for
// this translation unit.  The text and its length come straight from page-locked host memory the
// device can read (no copy node in front of the kernel), and the ids go straight to page-locked host
// memory (none behind it).
#define GTOK_COHERENT_LOADS 1
#include <cuda_runtime.h>
#include <stdint.h>

#include "encode_core.h"
#include "encode_kernels.h"
#include "gpu_block.cuh"

namespace gtok {

namespace {

union TinySmem {
    PretokSmem pretok;
    WordsSmem words;
    MissSmem miss;
    AsmSmem assemble;
};

// host_text / host_meta: device-visible addresses of page-locked host memory holding the text
// (padded to a multiple of 16 bytes) and {byte count, 1}; a.text / a.meta: the device buffers the
// tile programs work on, filled here.
__global__ void __launch_bounds__(kThreads, 1) tiny_kernel(const __grid_constant__ EncodeArgs a, const uint8_t* host_text, const uint32_t* host_meta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TinySmem& sm = *reinterpret_cast<TinySmem*>(smem_raw);
    GpuBlk blk;
    const int tid = threadIdx.x;
    const uint32_t n = host_meta[0] <= kTinyMaxBytes ? host_meta[0] : 0u;
    tl_stamp(a, 5, 0);
    // the text into device memory, the control words and per-tile counters to zero
    {
        const uint32_t quads = (n + 15u) / 16u;
        const uint4* src = reinterpret_cast<const uint4*>(host_text);
        uint4* dst = reinterpret_cast<uint4*>(const_cast<uint8_t*>(a.text));
        for (uint32_t i = tid; i < quads; i += kThreads) dst[i] = src[i];
        if (tid < 16) a.ctl[tid] = 0;
        if (tid == 0) { const_cast<uint32_t*>(a.meta)[0] = n; const_cast<uint32_t*>(a.meta)[1] = 1; }
        const uint32_t tiles = n / kTile + 2;
        for (uint32_t i = tid; i < tiles; i += kThreads) { a.tile_tok[i] = 0; a.st1[i] = 0; a.st2[i] = 0; }
    }
    __syncthreads();
    tl_stamp(a, 5, 1);
    if (n == 0) { if (tid == 0) { a.status[0] = 0; a.status[1] = host_meta[0] ? kErrInternal : 0u; } return; }
    const int p_tiles = static_cast<int>((n + kPTile - 1) / kPTile), w_tiles = static_cast<int>((n + kTile - 1) / kTile);
    if (a.tb.uc_wide) {
        pretok_block_init<true>(blk, a, sm.pretok);
        for (int t = 0; t < p_tiles; ++t) {
            if (tid == 0) sm.pretok.misc[2] = 2;        // no timeline row for this kernel
            pretok_tile<true>(blk, a, sm.pretok, t);
        }
    } else {
        pretok_block_init<false>(blk, a, sm.pretok);
        for (int t = 0; t < p_tiles; ++t) {
            if (tid == 0) sm.pretok.misc[2] = 2;
            pretok_tile<false>(blk, a, sm.pretok, t);
        }
    }
    __syncthreads();
    tl_stamp(a, 5, 2);
    for (int t = 0; t < w_tiles; ++t) words_tile(blk, a, sm.words, t);
    __syncthreads();
    tl_stamp(a, 5, 3);
    {
        MissSmem& ms = sm.miss;
        // every unknown pre-token of 2..64 bytes is in the one list (a.one_list): batches as large as the
        // longest of them allows, so that a short prompt's merge loops all run side by side
        const uint32_t n_miss = a.ctl[CTL_NMISS], n_long = a.ctl[CTL_NLONG];
        __shared__ uint32_t s_maxlen;
        if (tid == 0) s_maxlen = 0;
        ms.b2i[tid] = a.tb.byte_to_id[tid];
        __syncthreads();
        {
            uint32_t mx = 0;
            for (uint32_t i = tid; i < n_miss; i += kThreads) mx = max(mx, static_cast<uint32_t>(a.gmiss[i] >> 32));
            if (mx) atomicMax(&s_maxlen, mx);
        }
        __syncthreads();
        const uint32_t longest = s_maxlen;
        uint32_t batch = kMissBatch, max_len = kShortWordMax;
        if (longest > static_cast<uint32_t>(kMedSplit1)) { batch = kMedBatchA; max_len = kMedWordMax; }
        else if (longest > static_cast<uint32_t>(kMedSplit)) { batch = kMedBatchA1; max_len = kMedSplit1; }
        else if (longest > static_cast<uint32_t>(kShortWordMax)) { batch = kMedBatchB; max_len = kMedSplit; }
        // (no more arena than there are entries: the fetch and pair phases pass over batch * max_len slots)
        if (n_miss < batch) batch = n_miss ? (n_miss + 3u) & ~3u : 4u;
        for (uint32_t first = 0; first < n_miss; first += batch) miss_batch(blk, a, ms, a.gmiss, 1, first, n_miss, batch, max_len, batch);
        for (uint32_t li = 0; li < n_long; ++li) long_word(blk, a, ms, li);
    }
    __syncthreads();
    tl_stamp(a, 5, 4);
    for (int t = 0; t < w_tiles; ++t) assemble_tile(blk, a, sm.assemble, t);
    __syncthreads();
    tl_stamp(a, 5, 5);
    if (tid == 0) {
        __threadfence_system();
        a.status[1] = a.ctl[CTL_ERR];
    }
}

}  // namespace

cudaError_t configure_tiny_kernel() {
    cudaError_t e = cudaFuncSetAttribute(tiny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(TinySmem)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tiny_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return e;
}

void launch_tiny(const EncodeArgs& a, const uint8_t* host_text, const uint32_t* host_meta, cudaStream_t s) {
    tiny_kernel<<<1, kThreads, sizeof(TinySmem), s>>>(a, host_text, host_meta);
}

}  // namespace gtok
