// CUDA kernels of the encode path for sm_100a: thin persistent wrappers around the
// tile programs of encode_core.h, plus the launch helpers the engine captures into
// its CUDA graph.
//
// Both kernels are persistent: a fixed grid (a multiple of the SM count) pulls tile
// numbers from a ticket counter, so the work done depends on the byte count that
// sits in device memory, not on the capacity the graph was captured for, and a tile
// never waits on a tile that has not been handed to a running block.
#include <cuda_runtime.h>
#include <stdint.h>

#include "encode_core.h"
#include "encode_kernels.h"

namespace gtok {

namespace {

struct GpuBlk {
    template <class F>
    __device__ __forceinline__ void par(F f) {
        f(static_cast<int>(threadIdx.x));
        __syncthreads();
    }
    // In-place exclusive scan of arr[kThreads] (shared memory); every thread gets the total.
    __device__ __forceinline__ void excl_scan(uint32_t* arr, uint32_t* total) {
        __shared__ uint32_t wsum[kThreads / 32];
        const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
        const uint32_t v = arr[tid];
        uint32_t x = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t y = __shfl_up_sync(0xFFFFFFFFu, x, d);
            if (lane >= d) x += y;
        }
        if (lane == 31) wsum[wid] = x;
        __syncthreads();
        uint32_t off = 0, tot = 0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            uint32_t s = wsum[w];
            if (w < wid) off += s;
            tot += s;
        }
        arr[tid] = off + x - v;
        *total = tot;
        __syncthreads();
    }
    __device__ __forceinline__ uint32_t reduce_min(uint32_t* arr) {
        __shared__ uint32_t wmin[kThreads / 32];
        const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
        uint32_t x = __reduce_min_sync(0xFFFFFFFFu, arr[tid]);
        if (lane == 0) wmin[wid] = x;
        __syncthreads();
        uint32_t m = 0xFFFFFFFFu;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) m = min(m, wmin[w]);
        __syncthreads();
        return m;
    }
};

__global__ void __launch_bounds__(kThreads) pretok_kernel(const EncodeArgs a) {
    __shared__ PretokSmem sm;
    __shared__ int s_tile;
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kTile - 1) / kTile);
    for (;;) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + 0, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        pretok_tile(blk, a, sm, tile);
    }
}

__global__ void __launch_bounds__(kThreads) merge_kernel(const EncodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    MergeSmem& sm = *reinterpret_cast<MergeSmem*>(smem_raw);
    __shared__ int s_tile;
    GpuBlk blk;
    const uint32_t n = a.meta[0];
    const int n_tiles = static_cast<int>((n + kTile - 1) / kTile);
    for (;;) {
        if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(a.ctl + 1, 1u));
        __syncthreads();
        const int tile = s_tile;
        __syncthreads();
        if (tile >= n_tiles) break;
        merge_tile(blk, a, sm, tile);
    }
    // The last block to leave mirrors the error word where the host can read it.
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.ctl + 3, 1u) == gridDim.x - 1) {
            __threadfence();
            a.status[1] = *reinterpret_cast<volatile uint32_t*>(a.ctl + 2);
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

}  // namespace

size_t merge_smem_bytes() { return sizeof(MergeSmem); }

cudaError_t configure_kernels() {
    return cudaFuncSetAttribute(merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(MergeSmem)));
}

int pretok_blocks_per_sm() {
    int nb = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, pretok_kernel, kThreads, 0);
    return nb > 0 ? nb : 1;
}
int merge_blocks_per_sm() {
    int nb = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, merge_kernel, kThreads, sizeof(MergeSmem));
    return nb > 0 ? nb : 1;
}

void launch_docmask(const EncodeArgs& a, uint32_t* docmask, int blocks, cudaStream_t s) {
    docmask_kernel<<<blocks, 256, 0, s>>>(a.meta, a.doc_off, docmask);
}
void launch_pretok(const EncodeArgs& a, int blocks, cudaStream_t s) { pretok_kernel<<<blocks, kThreads, 0, s>>>(a); }
void launch_merge(const EncodeArgs& a, int blocks, cudaStream_t s) {
    merge_kernel<<<blocks, kThreads, sizeof(MergeSmem), s>>>(a);
}

}  // namespace gtok
