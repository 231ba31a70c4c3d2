// CUDA kernels of the encode path for sm_100a: thin persistent wrappers around the
// tile programs of encode_core.h, plus the launch helpers the engine captures into
// its CUDA graph.
//
// The kernels are persistent: a fixed grid (a multiple of the SM count) walks the tiles,
// so the work done depends on the byte count that sits in device memory, not on the
// capacity the graph was captured for.  Where a tile waits on earlier tiles (look-back)
// tiles are handed out by a ticket counter, so a tile never waits on one no block has started.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "encode_core.h"
#include "decode_core.h"
#include "encode_kernels.h"
#include "gpu_block.cuh"
#include "nfc_core.h"

namespace gtok {

namespace {

template <bool kWide>
__device__ __forceinline__ void pretok_body(const EncodeArgs& a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PretokSmem& sm = *reinterpret_cast<PretokSmem*>(smem_raw);
    __shared__ int s_tile;
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kPTile - 1) / kPTile);
    tl_stamp(a, 0, 0);
    pretok_block_init<kWide>(blk, a, sm);
    for (int done = 0;; ++done) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + 0, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        if (threadIdx.x == 0) sm.misc[2] = static_cast<uint32_t>(done);      // diagnostics: which of the block's tiles this is
        pretok_tile<kWide>(blk, a, sm, tile);
        tl_stamp(a, 0, 2 + done);
    }
    tl_stamp(a, 0, 1);
}
__global__ void __launch_bounds__(kThreads, 4) pretok_kernel(const __grid_constant__ EncodeArgs a) { pretok_body<false>(a); }
// The same for vocabularies of the DeepSeek-V3 family (wide class table, its own rules): a kernel of its own, so
// that neither family's code weighs on the other's registers.
__global__ void __launch_bounds__(kThreads, 4) pretok_wide_kernel(const __grid_constant__ EncodeArgs a) { pretok_body<true>(a); }

// Kernel 0 (vocabularies that declare NFC): raw text -> normalised text, byte count and
// document offsets; tiles in ticket order because a tile's place in the output is the sum of
// the lengths of all earlier tiles.
// Does the text need normalising at all?  Any codepoint that can make a text non-NFC raises the
// flag.  (Launched with raw_docmask unset: document boundaries are ignored here, which can only
// raise the flag once too often.)
__global__ void __launch_bounds__(kThreads) nfc_check_kernel(const __grid_constant__ EncodeArgs a) {
    const uint32_t n = a.raw_meta[0];
    if (a.raw_meta[2]) return;                                   // the host says it is normalised already
    const uint32_t chunks = (n + kPer - 1) / kPer;
    uint32_t any = 0;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += gridDim.x * blockDim.x) {
        uint32_t l, f;
        nfc_chunk_masks(a, static_cast<long long>(c) * kPer, n, &l, &f);
        any |= l;
    }
    if (__syncthreads_or(any != 0) && threadIdx.x == 0) atomicOr(a.ctl + CTL_NFCFLAG, 1u);
}

// Nothing to normalise (the usual case): the raw text and its header are the text and the header.
__global__ void __launch_bounds__(kThreads) nfc_copy_kernel(const __grid_constant__ EncodeArgs a) {
    if (a.ctl[CTL_NFCFLAG]) return;
    const uint32_t n = a.raw_meta[0], n_docs = a.raw_meta[1];
    const uint32_t quads = (n + 15) / 16;
    const uint4* src = reinterpret_cast<const uint4*>(a.raw);
    uint4* dst = reinterpret_cast<uint4*>(a.norm_text);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += gridDim.x * blockDim.x) dst[i] = src[i];
    const uint32_t hdr = 4u + (a.raw_doc_off ? n_docs + 1u : 0u);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < hdr; i += gridDim.x * blockDim.x) a.norm_meta[i] = a.raw_meta[i];
    if (blockIdx.x == 0 && threadIdx.x == 0) a.status[2] = n;
}

__global__ void __launch_bounds__(kThreads) nfc_kernel(const __grid_constant__ EncodeArgs a) {
    __shared__ NfcSmem sm;
    __shared__ int s_tile;
    GpuBlk blk;
    if (!a.ctl[CTL_NFCFLAG]) return;                             // nothing to normalise: the copy kernel has moved the text over
    const uint32_t n = a.raw_meta[0];
    const int n_tiles = static_cast<int>((n + kTile - 1) / kTile);
    for (;;) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + CTL_NFC, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        nfc_tile(blk, a, sm, tile);
    }
}

// Kernel 2: whole-word table lookups, tile by tile (tiles are independent here).
__global__ void __launch_bounds__(kThreads, 4) words_kernel(const __grid_constant__ EncodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    WordsSmem& sm = *reinterpret_cast<WordsSmem*>(smem_raw);
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kTile - 1) / kTile);
    tl_stamp(a, 1, 0);
    int done = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) { words_tile(blk, a, sm, tile); tl_stamp(a, 1, 2 + done++); }
    tl_stamp(a, 1, 1);
}

// Kernel 3: merge loops for what the table did not know, batch by batch, then the
// pre-tokens longer than 64 bytes one by one.
__global__ void __launch_bounds__(kThreads, 4) miss_kernel(const __grid_constant__ EncodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    MissSmem& sm = *reinterpret_cast<MissSmem*>(smem_raw);
    __shared__ uint32_t s_pick;
    GpuBlk blk;
    const uint32_t n_miss = a.ctl[CTL_NMISS], n_med = a.ctl[CTL_NMED], n_med1 = a.ctl[CTL_NMED1], n_med2 = a.ctl[CTL_NMED2], n_long = a.ctl[CTL_NLONG];
    const uint32_t take_b = a.tb.ignore_merges ? kMedTakeB : kMedBatchB;      // list entries per call of the 17..32-byte class
    const uint32_t med2_batches = (n_med2 + take_b - 1) / take_b;
    const uint32_t short_batches = (n_miss + kMissBatch - 1) / kMissBatch;
    // Pre-tokens per call of the two longest classes: an arena's worth, unless that leaves most blocks without a call (a
    // prompt, a shard of a document): then a quarter, so that a call's fetch and pair phases, which the merge chains wait for,
    // are a quarter as long.
    uint32_t batch_a = kMedBatchA, batch_a1 = kMedBatchA1;
    if (2u * ((n_med + kMedBatchA / 4 - 1) / (kMedBatchA / 4) + (n_med1 + kMedBatchA1 / 4 - 1) / (kMedBatchA1 / 4) + med2_batches + short_batches + n_long) < gridDim.x) {
        batch_a = kMedBatchA / 4;
        batch_a1 = kMedBatchA1 / 4;
    }
    const uint32_t med_batches = (n_med + batch_a - 1) / batch_a, med1_batches = (n_med1 + batch_a1 - 1) / batch_a1;
    // A call of the 17..32-byte class under ignore_merges looks 256 entries up as whole tokens but merges at most 96
    // of them at a time.  With fewer calls than blocks (a prompt rather than a corpus) it hands the rest back for the
    // blocks that got no call; otherwise it works through the rest itself, which keeps the blocks evenly loaded.
    const bool share = take_b > kMedBatchB && med2_batches != 0 && med_batches + med1_batches + med2_batches + short_batches + n_long < gridDim.x;
    tl_stamp(a, 2, 0);
    sm.b2i[threadIdx.x] = a.tb.byte_to_id[threadIdx.x];
    __syncthreads();
    // the pre-tokens of more than 64 bytes first, a block each (the longest of them take longer than a block's share of
    // the batches), then the batches, longest class first: their merge chains decide when the kernel ends
    for (;;) {
        if (threadIdx.x == 0) s_pick = atomicAdd(a.ctl + CTL_LONG, 1u);
        __syncthreads();
        const uint32_t li = s_pick;
        __syncthreads();
        if (li >= n_long) break;
        long_word(blk, a, sm, li);
    }
    for (int done = 0;; ++done) {
        if (threadIdx.x == 0) s_pick = atomicAdd(a.ctl + CTL_BATCH, 1u);
        __syncthreads();
        const uint32_t t = s_pick;
        __syncthreads();
        if (t >= med_batches + med1_batches + med2_batches + short_batches) break;
        const unsigned long long* list = a.gmiss;
        int dir = 1;
        uint32_t first = (t - med_batches - med1_batches - med2_batches) * kMissBatch, count = n_miss, batch = kMissBatch, max_len = kShortWordMax, take = kMissBatch;
        if (t < med_batches) { list = a.gmed; first = t * batch_a; count = n_med; batch = batch_a; max_len = kMedWordMax; take = batch_a; }
        else if (t < med_batches + med1_batches) { list = a.gmed1; first = (t - med_batches) * batch_a1; count = n_med1; batch = batch_a1; max_len = kMedSplit1; take = batch_a1; }
        else if (t < med_batches + med1_batches + med2_batches) {
            list = a.gmed + (a.gmed_cap - 1); dir = -1; first = (t - med_batches - med1_batches) * take_b; count = n_med2; batch = kMedBatchB; max_len = kMedSplit; take = take_b;
        }
        if (share && take > batch) miss_batch_sharing(blk, a, sm, list, dir, first, count, batch, max_len, take);
        else miss_batch(blk, a, sm, list, dir, first, count, batch, max_len, take);
        tl_stamp(a, 2, 2 + done);
    }
    // What the calls of the 17..32-byte class handed back: wait until every such call is through its lookups, then
    // take the chunks in turn.  The wait is for blocks that are running (a call is only ever held by a block that
    // took its ticket).
    if (share) {
        if (threadIdx.x == 0)
            s_pick = wait_count(a.ctl + CTL_FILTERED, med2_batches, a.ctl) && *reinterpret_cast<volatile uint32_t*>(a.ctl + CTL_NSURPLUS) ? 1u : 0u;   // usually nothing
        __syncthreads();
        const bool ready = s_pick != 0;
        __syncthreads();
        while (ready) {
            if (threadIdx.x == 0) s_pick = atomicAdd(a.ctl + CTL_SURPLUS, 1u);
            __syncthreads();
            const uint32_t u = s_pick;
            __syncthreads();
            if (u >= med2_batches * kSurplusChunks) break;
            miss_surplus(blk, a, sm, a.gmed + (a.gmed_cap - 1), -1, (u / kSurplusChunks) * take_b, u % kSurplusChunks);
        }
    }
    tl_stamp(a, 2, 1);
}

// Kernel 4: output assembly; tiles are handed out in order because a tile's base is the
// sum of all earlier tiles' counts.
__global__ void __launch_bounds__(kThreads, 8) assemble_kernel(const __grid_constant__ EncodeArgs a) {
    __shared__ AsmSmem sm;
    __shared__ int s_tile;
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kTile - 1) / kTile);
    tl_stamp(a, 3, 0);
    for (int done = 0;; ++done) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + CTL_ASM, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        assemble_tile(blk, a, sm, tile);
        tl_stamp(a, 3, 2 + done);
    }
    tl_stamp(a, 3, 1);
    // The last block to leave mirrors the error word where the host can read it.
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.ctl + CTL_EXIT, 1u) == gridDim.x - 1) {
            __threadfence();
            a.status[1] = *reinterpret_cast<volatile uint32_t*>(a.ctl + CTL_ERR);
        }
    }
}

// One bit per byte, set where a document of the batch begins.
__global__ void docmask_kernel(const uint32_t* meta, const uint32_t* doc_off, uint32_t* docmask) {
    const uint32_t n = meta[0], n_docs = meta[1];
    for (uint32_t d = blockIdx.x * blockDim.x + threadIdx.x; d <= n_docs; d += gridDim.x * blockDim.x) {
        uint32_t off = doc_off[d];
        if (off < n) atomicOr(docmask + (off >> 5), 1u << (off & 31));
    }
}

// ---- boundaries without any allocation --------------------------------------------
// Working memory of boundaries_noalloc(): the pre-tokenization kernel's ticket and error
// words, its per-tile look-back states, the per-tile boundary counts, the added-token
// bits and the byte count the kernel reads.  It lives in the library's device image:
// every GPU that loads the library holds these ~0.5 MB until the process exits.
struct NoAllocScratch {
    uint32_t ctl[16];
    uint32_t meta[16];
    unsigned long long st1[kNoAllocTiles + 1];
    uint32_t tile_nb[kNoAllocTiles + 1];
    uint32_t amask[kNoAllocTiles * kTileWords + 8];
};
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

__global__ void noalloc_set_meta(uint32_t* meta, uint32_t n) { meta[0] = n; meta[1] = 1; }

}  // namespace

int boundaries_noalloc(const DeviceTables& tb, int device, const void* text_dev, uint32_t len, void* out_bits_dev,
                       cudaStream_t stream, std::string& err) {
    if (len > kNoAllocMaxBytes) {
        err = "boundaries_noalloc: input of " + std::to_string(len) + " bytes exceeds the fixed working memory (limit " +
              std::to_string(kNoAllocMaxBytes) + " bytes)";
        return -3;
    }
    if (!text_dev || !out_bits_dev) { err = "boundaries_noalloc: null device pointer"; return -1; }
    if (reinterpret_cast<uintptr_t>(text_dev) & 15u) { err = "boundaries_noalloc: text must be 16-byte aligned"; return -1; }
    if (len == 0) return 0;
    // Device address of the scratch array, looked up once per device with that device
    // current.  In host code the array's name is only a handle for this lookup.
    static std::mutex mu;
    static NoAllocScratch* scratch_of[64] = {};
    static int sm_of[64] = {};
    if (device < 0 || device >= 64) { err = "boundaries_noalloc: device index out of range"; return -1; }
    // The handle's device becomes current for the duration of the call only: the caller's own
    // current device is put back on every way out.
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    } guard;
    int was = -1;
    if (cudaGetDevice(&was) != cudaSuccess) was = -1;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { err = std::string("cudaSetDevice: ") + cudaGetErrorString(e); return -1; }
    if (was >= 0 && was != device) guard.prev = was;
    NoAllocScratch* sc;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_of[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) { err = std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e); return -1; }
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess || sms <= 0) { err = std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e); return -1; }
            sm_of[device] = sms;
            scratch_of[device] = static_cast<NoAllocScratch*>(p);
        }
        sc = scratch_of[device];
    }
    EncodeArgs a;
    memset(&a, 0, sizeof a);
    a.text = static_cast<const uint8_t*>(text_dev);
    a.meta = sc->meta;
    a.bmask = static_cast<uint32_t*>(out_bits_dev);
    a.amask = sc->amask;
    a.tile_nb = sc->tile_nb;
    a.st1 = sc->st1;
    a.ctl = sc->ctl;
    a.tb = tb;
    const uint32_t n_tiles = (len + kPTile - 1) / kPTile;      // tiles of the pre-tokenization kernel
    // The array keeps whatever the previous call left: ticket, error word and the
    // look-back states of the tiles this call uses must start at zero.
    e = cudaMemsetAsync(sc->ctl, 0, sizeof sc->ctl, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(sc->st1, 0, sizeof(unsigned long long) * (n_tiles + 1), stream);
    if (e != cudaSuccess) { err = std::string("cudaMemsetAsync: ") + cudaGetErrorString(e); return -1; }
    noalloc_set_meta<<<1, 1, 0, stream>>>(sc->meta, len);
    const int blocks = static_cast<int>(n_tiles < static_cast<uint32_t>(sm_of[device] * 4) ? n_tiles : sm_of[device] * 4);
    if (a.tb.uc_wide) pretok_wide_kernel<<<blocks, kThreads, sizeof(PretokSmem), stream>>>(a);
    else pretok_kernel<<<blocks, kThreads, sizeof(PretokSmem), stream>>>(a);
    e = cudaGetLastError();
    // The kernel's error word comes back with the result (a copy into a local variable: no
    // allocation).  A wait on an earlier tile that gave up leaves wrong bits behind, and two calls
    // that overlapped on the shared array can end that way: both must fail, not return 0.
    uint32_t err_bits = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&err_bits, sc->ctl + CTL_ERR, sizeof err_bits, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { err = std::string("boundaries_noalloc: ") + cudaGetErrorString(e); return -1; }
    if (err_bits) {
        char buf[112];
        std::snprintf(buf, sizeof buf, "boundaries_noalloc: the kernel reported error bits 0x%x (0x2 = a wait on an earlier tile gave up)", err_bits);
        err = buf;
        return -1;
    }
    return 0;
}

cudaError_t configure_kernels() {
    cudaError_t e = cudaFuncSetAttribute(words_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(WordsSmem)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(pretok_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PretokSmem)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(pretok_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(pretok_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PretokSmem)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(pretok_wide_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(assemble_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(miss_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(MissSmem)));
    // All four kernels work out of shared memory, not L1: the largest carve-out for each, so that as
    // many blocks as the register file allows are resident and the SMs keep one configuration
    // from kernel to kernel of a replay.
    if (e == cudaSuccess) e = cudaFuncSetAttribute(words_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(miss_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return e;
}

// Decoding kernel: tiles of 2048 ids handed out in order (a tile's byte offset is the sum of
// the earlier tiles' byte counts, found by look-back).
__global__ void __launch_bounds__(kThreads, 4) decode_kernel(const __grid_constant__ DecodeArgs a) {
    __shared__ DecodeSmem sm;
    __shared__ int s_tile;
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kDecIds - 1) / kDecIds);
    for (;;) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + CTL_PRETOK, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        decode_tile(blk, a, sm, tile);
    }
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.ctl + CTL_EXIT, 1u) == gridDim.x - 1) {
            __threadfence();
            if (n == 0) a.status[0] = 0;
            a.status[1] = *reinterpret_cast<volatile uint32_t*>(a.ctl + CTL_ERR);
        }
    }
}

static int blocks_per_sm(const void* fn, size_t smem) {
    int nb = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fn, kThreads, smem);
    return nb > 0 ? nb : 1;
}
int pretok_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(pretok_kernel), sizeof(PretokSmem)); }
int words_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(words_kernel), sizeof(WordsSmem)); }
int miss_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(miss_kernel), sizeof(MissSmem)); }
int nfc_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(nfc_kernel), 0); }
int decode_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(decode_kernel), 0); }
int assemble_blocks_per_sm() { return blocks_per_sm(reinterpret_cast<const void*>(assemble_kernel), 0); }

void launch_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s) {
    docmask_kernel<<<blocks, 256, 0, s>>>(a.meta, a.doc_off, docmask);
}
void launch_raw_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s) {
    docmask_kernel<<<blocks, 256, 0, s>>>(a.raw_meta, a.raw_doc_off, docmask);
}
void launch_nfc_check(const EncodeArgs& a, int blocks, cudaStream_t s) { nfc_check_kernel<<<blocks, kThreads, 0, s>>>(a); }
void launch_nfc_copy(const EncodeArgs& a, int blocks, cudaStream_t s) { nfc_copy_kernel<<<blocks, kThreads, 0, s>>>(a); }
void launch_nfc(const EncodeArgs& a, int blocks, cudaStream_t s) { nfc_kernel<<<blocks, kThreads, 0, s>>>(a); }
void launch_pretok(const EncodeArgs& a, int blocks, cudaStream_t s) {
    if (a.tb.uc_wide) pretok_wide_kernel<<<blocks, kThreads, sizeof(PretokSmem), s>>>(a);
    else pretok_kernel<<<blocks, kThreads, sizeof(PretokSmem), s>>>(a);
}
const void* words_kernel_address() { return reinterpret_cast<const void*>(words_kernel); }
const void* miss_kernel_address() { return reinterpret_cast<const void*>(miss_kernel); }
void launch_words(const EncodeArgs& a, int blocks, cudaStream_t s) { words_kernel<<<blocks, kThreads, sizeof(WordsSmem), s>>>(a); }
void launch_miss(const EncodeArgs& a, int blocks, cudaStream_t s) { miss_kernel<<<blocks, kThreads, sizeof(MissSmem), s>>>(a); }
void launch_decode(const DecodeArgs& a, int blocks, cudaStream_t s) { decode_kernel<<<blocks, kThreads, 0, s>>>(a); }
void launch_assemble(const EncodeArgs& a, int blocks, cudaStream_t s) { assemble_kernel<<<blocks, kThreads, 0, s>>>(a); }

}  // namespace gtok
