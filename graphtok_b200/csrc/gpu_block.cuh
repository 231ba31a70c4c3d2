// The "thread block" object the tile programs of encode_core.h are written against, for the GPU:
// one real thread per tid, barriers, warp-shuffle scans, the decoupled look-back.  Shared by the
// kernels of encode_kernels.cu and the single-block kernel of tiny_kernel.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "encode_core.h"

namespace gtok {

struct GpuBlk {
    // Per-thread values that live from one par() to the next: registers here.
    template <class T>
    struct Local {
        T v;
        __device__ __forceinline__ T& at(int) { return v; }
    };
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
    // excl_scan of arr[kThreads] and, in the same two barriers, the plain sum of other[kThreads].
    __device__ __forceinline__ void excl_scan_and_sum(uint32_t* arr, uint32_t* total, const uint32_t* other, uint32_t* other_total) {
        __shared__ uint32_t wsum2[kThreads / 32], osum2[kThreads / 32];
        const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
        const uint32_t v = arr[tid];
        uint32_t x = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t y = __shfl_up_sync(0xFFFFFFFFu, x, d);
            if (lane >= d) x += y;
        }
        const uint32_t o = __reduce_add_sync(0xFFFFFFFFu, other[tid]);
        if (lane == 31) wsum2[wid] = x;
        if (lane == 0) osum2[wid] = o;
        __syncthreads();
        uint32_t off = 0, tot = 0, otot = 0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            uint32_t s = wsum2[w];
            if (w < wid) off += s;
            tot += s;
            otot += osum2[w];
        }
        arr[tid] = off + x - v;
        *total = tot;
        *other_total = otot;
        __syncthreads();
    }
    // Publishes this tile's total and returns the sum of all earlier tiles' totals: warp 0
    // reads 32 predecessors' states at a time, adds them up to the nearest one whose value
    // already includes everything before it.
    __device__ __forceinline__ uint32_t lookback(unsigned long long* st, int tile, uint32_t total, uint32_t* ctl) {
        __shared__ uint32_t s_base;
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            if (lane == 0) store_state(st + tile, (tile == 0 ? kStFinal : kStAgg) | total);
            // (sums saturate at 0xFFFFFFFF instead of wrapping: a total of 4 GiB or more stays visible to every later tile)
            unsigned long long base = 0;
            int hi = tile - 1;
            bool done = tile == 0;
            while (!done) {
                const int j = hi - lane;
                unsigned long long v = kStFinal;
                if (j >= 0) v = wait_state(st, j, ctl);
                const unsigned fin = __ballot_sync(0xFFFFFFFFu, (v >> 62) == 2);
                uint32_t val = static_cast<uint32_t>(v);
                if (fin) {
                    const int first = __ffs(fin) - 1;
                    if (lane > first) val = 0;
                    done = true;
                }
                base += (static_cast<unsigned long long>(__reduce_add_sync(0xFFFFFFFFu, val >> 16)) << 16) + __reduce_add_sync(0xFFFFFFFFu, val & 0xFFFFu);
                hi -= 32;
            }
            if (base > 0xFFFFFFFFull) base = 0xFFFFFFFFull;
            if (lane == 0) {
                const unsigned long long incl = base + total > 0xFFFFFFFFull ? 0xFFFFFFFFull : base + total;
                if (tile > 0) store_state(st + tile, kStFinal | incl);
                s_base = static_cast<uint32_t>(base);
            }
        }
        __syncthreads();
        const uint32_t b = s_base;
        __syncthreads();
        return b;
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

// Diagnostics: a stamp of the global nanosecond timer in this block's row of the timeline.
__device__ __forceinline__ void tl_stamp(const EncodeArgs& a, int kernel, int slot) {
    if (!a.phase_clk || threadIdx.x != 0 || blockIdx.x >= kTlBlocks || slot >= kTlSlots) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.phase_clk[kPhaseWords + (static_cast<size_t>(kernel) * kTlBlocks + blockIdx.x) * kTlSlots + slot] = t;
}

}  // namespace gtok
