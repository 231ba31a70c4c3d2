// Decoding: token ids -> the bytes they spell, as one tile program.
//
//   decode_tile : 2048 ids -> their spellings at their final place in the output.
//
// Behaviour follows the reference's decode path (src/tokenizer.cu:5225-5275: per-id length,
// exclusive sum, gather of the vocabulary's byte strings; host side src/tokenizer.cu:5499-5573),
// as one pass instead of three launches: lengths, a block scan, a decoupled look-back across
// tiles for the tile's byte offset, then the gather through shared memory so that the output is
// written with aligned 16-byte stores whatever the tokens' lengths are.
//
// Written against the same "thread block" interface as the encoder's tile programs
// (encode_core.h), so that the CUDA kernel and the serial emulation of the CPU tests run the
// same code.  An id outside the vocabulary spells nothing and sets kErrBadId (the reference
// indexes its tables with it unchecked).
#pragma once
#include <stdint.h>

#include "encode_core.h"

namespace gtok {

constexpr int kDecPer = 8;                         // ids per thread
constexpr int kDecIds = kThreads * kDecPer;        // ids per tile
constexpr int kDecBuf = 16384;                     // output bytes staged per round (a multiple of 16)

enum : uint32_t { kErrBadId = 64u };               // joins the error bits of encode_core.h

struct DecodeArgs {
    const uint32_t* ids;
    const uint32_t* meta;            // [0] = number of ids
    const uint32_t* tok_off;         // [vocab_size + 1] offsets of the spellings in `blob`
    const uint8_t* blob;
    const uint32_t* tok16;           // [vocab_size][4]: the first 16 bytes of every spelling, one aligned load per id
    uint32_t vocab_size;
    unsigned long long* st;          // look-back state per tile
    uint32_t* ctl;                   // CTL_PRETOK = ticket, CTL_ERR, CTL_EXIT as in the encoder
    uint8_t* out;                    // 16-byte aligned
    uint32_t out_cap;
    uint32_t* status;                // [0] = bytes, [1] = error bits (host-visible)
};

struct DecodeSmem {
    uint32_t scan[kThreads];
    uint32_t id[kDecIds];            // the ids (those outside the vocabulary replaced by 0, with no bytes)
    uint32_t dst[kDecIds + 1];       // offset of each id's bytes in the tile's output
    alignas(16) uint8_t buf[kDecBuf + 16];
};

template <class Blk>
GTOK_DEV void decode_tile(Blk& blk, const DecodeArgs& a, DecodeSmem& sm, int tile) {
    const uint32_t n = ldg(a.meta);
    const uint32_t i0 = static_cast<uint32_t>(tile) * kDecIds;
    const uint32_t n_tiles = (n + kDecIds - 1) / kDecIds;
    // ---- D0: lengths ----
    blk.par([&](int tid) {
        const uint32_t first = i0 + tid * kDecPer;
        uint32_t id[kDecPer];
#if defined(__CUDA_ARCH__)
        if (first + kDecPer <= n) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(a.ids + first));
            const uint4 y = __ldg(reinterpret_cast<const uint4*>(a.ids + first) + 1);
            id[0] = x.x; id[1] = x.y; id[2] = x.z; id[3] = x.w;
            id[4] = y.x; id[5] = y.y; id[6] = y.z; id[7] = y.w;
        } else
#endif
        {
            for (int k = 0; k < kDecPer; ++k) id[k] = first + k < n ? ldg(a.ids + first + k) : 0xFFFFFFFFu;
        }
        uint32_t lo[kDecPer], hi[kDecPer];
        bool bad = false;
#pragma unroll
        for (int k = 0; k < kDecPer; ++k) {
            const bool in = id[k] < a.vocab_size;
            bad |= !in && first + k < n;
            lo[k] = in ? ldg(a.tok_off + id[k]) : 0u;
            hi[k] = in ? ldg(a.tok_off + id[k] + 1) : 0u;
        }
        uint32_t sum = 0;
#pragma unroll
        for (int k = 0; k < kDecPer; ++k) {
            sm.id[tid * kDecPer + k] = id[k] < a.vocab_size ? id[k] : 0u;
            sm.dst[tid * kDecPer + k] = sum;      // relative to the thread's first byte for now
            sum += hi[k] - lo[k];
        }
        sm.scan[tid] = sum;
        if (bad) global_or(a.ctl + CTL_ERR, kErrBadId);
    });
    uint32_t total = 0;
    blk.excl_scan(sm.scan, &total);
    blk.par([&](int tid) {
        const uint32_t at = sm.scan[tid];
#pragma unroll
        for (int k = 0; k < kDecPer; ++k) sm.dst[tid * kDecPer + k] += at;
        if (tid == kThreads - 1) sm.dst[kDecIds] = total;
    });
    // ---- D1: the tile's place in the output ----
    const uint32_t base = blk.lookback(a.st, tile, total, a.ctl);
    if (static_cast<uint32_t>(tile) + 1 == n_tiles) {
        blk.par([&](int tid) {
            if (tid == 0) a.status[0] = base + total < base ? 0xFFFFFFFFu : base + total;     // 0xFFFFFFFF: 4 GiB or more
        });
    }
    if (base + total > a.out_cap || base + total < base || base == 0xFFFFFFFFu) {
        blk.par([&](int tid) {
            if (tid == 0) global_or(a.ctl + CTL_ERR, kErrOutputFull);
        });
        return;
    }
    // ---- D2: gather, kDecBuf output bytes per round ----
    // Rounds are cut on 16-byte lines of the output: byte g of the output sits at buf[g - w0].
    const uint32_t end = base + total;
    for (uint32_t w0 = base & ~15u; w0 < end; w0 += kDecBuf) {
        const uint32_t w1 = w0 + kDecBuf < end ? w0 + kDecBuf : end;
        blk.par([&](int tid) {
            const uint32_t f = tid * kDecPer;
            if (base + sm.dst[f + kDecPer] <= w0 || base + sm.dst[f] >= w1) return;
            // Spellings of up to 16 bytes that lie inside this round come from the 16-byte table, all
            // eight loads in flight together; the rest byte by byte from the blob.
            uint32_t v[kDecPer][4];
            uint32_t at[kDecPer], len[kDecPer];
#pragma unroll
            for (int k = 0; k < kDecPer; ++k) {
                const uint32_t g = base + sm.dst[f + k], ge = base + sm.dst[f + k + 1];
                at[k] = g - w0;
                len[k] = ge - g;
                const bool quick = len[k] - 1u < 16u && g >= w0 && ge <= w1;
                if (!quick && len[k]) len[k] |= 0x80000000u;
                v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0;
                if (quick) {
                    const uint32_t* t = a.tok16 + static_cast<size_t>(sm.id[f + k]) * 4;
#if defined(__CUDA_ARCH__)
                    const uint4 x = __ldg(reinterpret_cast<const uint4*>(t));
                    v[k][0] = x.x; v[k][1] = x.y; v[k][2] = x.z; v[k][3] = x.w;
#else
                    for (int q = 0; q < 4; ++q) v[k][q] = t[q];
#endif
                }
            }
#pragma unroll
            for (int k = 0; k < kDecPer; ++k) {
                if (len[k] & 0x80000000u) {
                    uint32_t g = base + sm.dst[f + k];
                    const uint32_t ge = base + sm.dst[f + k + 1];
                    uint32_t s = ldg(a.tok_off + sm.id[f + k]);
                    if (g < w0) { s += w0 - g; g = w0; }
                    const uint32_t stop = ge < w1 ? ge : w1;
                    for (; g < stop; ++g, ++s) sm.buf[g - w0] = ldg(a.blob + s);
                    continue;
                }
#pragma unroll
                for (int b = 0; b < 16; ++b)
                    if (static_cast<uint32_t>(b) < len[k]) sm.buf[at[k] + b] = static_cast<uint8_t>(v[k][b >> 2] >> (8 * (b & 3)));
            }
        });
        blk.par([&](int tid) {
            const uint32_t lines = (w1 - w0 + 15) >> 4;
            for (uint32_t c = tid; c < lines; c += kThreads) {
                const uint32_t g = w0 + (c << 4);
                if (g >= base && g + 16 <= end) {
#if defined(__CUDA_ARCH__)
                    *reinterpret_cast<uint4*>(a.out + g) = *reinterpret_cast<const uint4*>(sm.buf + (c << 4));
#else
                    for (int b = 0; b < 16; ++b) a.out[g + b] = sm.buf[(c << 4) + b];
#endif
                } else {
                    // a line shared with the neighbouring tile: only this tile's bytes
                    for (uint32_t b = 0; b < 16; ++b)
                        if (g + b >= base && g + b < end) a.out[g + b] = sm.buf[(c << 4) + b];
                }
            }
        });
    }
}

}  // namespace gtok
