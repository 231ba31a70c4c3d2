// Unicode Normalization Form C on the device, tile by tile, for vocabularies whose
// tokenizer.json declares {"type": "NFC"} (Qwen2.5).  It produces, byte for byte, what
// the host normaliser (nfc_host.cc) produces, which in turn plays the role of the
// reference's normalize_view_for_vocab (src/vocab.cc:1234-1668).
//
// A text can only fail to be NFC around "attention" codepoints: those with a non-zero
// combining class, those not equal to their own NFC, and those that can combine with what
// precedes them (all are U+0300 or above).  A maximal run of attention codepoints together
// with the one codepoint before it (when that is well-formed and in the same document) is a
// stretch; NFC of the text is the text with every stretch replaced by its own NFC.  So:
//
//   N1  every thread flags the attention codepoints of its 16 bytes (a table bit per codepoint);
//   N2  the thread in whose bytes a stretch begins normalises it (decompose, canonical order,
//       compose) to learn its new length; every thread counts the bytes it will emit;
//   N3  block scan + look-back over tiles give each thread its place in the output;
//   N4  bytes outside stretches are copied, stretches are written normalised, document
//       offsets (batch) and the byte count are rewritten for the kernels that follow.
//
// Text without attention codepoints costs one 16-byte load, a bit test and one 16-byte
// store per thread.  Written against the same block interface as encode_core.h so that the
// CPU tests run the very same code.
#pragma once
#include "encode_core.h"

namespace gtok {

constexpr int kNfcMaxCps = 96;       // decomposed codepoints of one stretch; longer ones are flagged (kErrNfcLong)

constexpr int kNfcStage = kTile + 528;      // bytes of a tile's output put together in shared memory before they go out
struct NfcSmem {
    alignas(16) uint8_t outb[kNfcStage];
    uint8_t sres[kThreads][12];      // the normalised form of the one stretch a chunk owns, kept from sizing to writing
    uint8_t slen[kThreads];          // its length; 0: not kept (no stretch, several, or longer than that)
    uint32_t scan[kThreads];
    uint16_t attl[kThreads + 2];     // per 16-byte chunk, one before and one after the tile: attention lead bytes
    uint16_t attf[kThreads + 2];     // ... and every byte of an attention codepoint
    uint16_t drop[kThreads];         // bytes of the chunk that belong to a stretch
    uint16_t own[kThreads];          // stretches that begin in the chunk
    unsigned long long clk_last;
};

GTOK_DEV bool raw_docstart(const EncodeArgs& a, uint32_t p) {
    return a.raw_docmask && ((ldg(a.raw_docmask + (p >> 5)) >> (p & 31)) & 1u);
}

// Strict UTF-8 decode at q: width, or 0 when the bytes are not a well-formed sequence that
// lies inside [0, n) and inside one document.
GTOK_DEV int nfc_decode(const EncodeArgs& a, uint32_t q, uint32_t n, uint32_t* cp) {
    const uint32_t b = ldg(a.raw + q);
    if (b < 0x80) { *cp = b; return 1; }
    int w = 0;
    uint32_t v = 0;
    if (b >= 0xC2 && b <= 0xDF) {
        if (q + 2 > n) return 0;
        const uint32_t b1 = ldg(a.raw + q + 1);
        if ((b1 & 0xC0) != 0x80) return 0;
        v = ((b & 0x1Fu) << 6) | (b1 & 0x3Fu);
        w = 2;
    } else if ((b & 0xF0) == 0xE0) {
        if (q + 3 > n) return 0;
        const uint32_t b1 = ldg(a.raw + q + 1), b2 = ldg(a.raw + q + 2);
        if ((b1 & 0xC0) != 0x80 || (b2 & 0xC0) != 0x80) return 0;
        v = ((b & 0x0Fu) << 12) | ((b1 & 0x3Fu) << 6) | (b2 & 0x3Fu);
        if (v < 0x800 || (v >= 0xD800 && v <= 0xDFFF)) return 0;
        w = 3;
    } else if (b >= 0xF0 && b <= 0xF4) {
        if (q + 4 > n) return 0;
        const uint32_t b1 = ldg(a.raw + q + 1), b2 = ldg(a.raw + q + 2), b3 = ldg(a.raw + q + 3);
        if ((b1 & 0xC0) != 0x80 || (b2 & 0xC0) != 0x80 || (b3 & 0xC0) != 0x80) return 0;
        v = ((b & 0x07u) << 18) | ((b1 & 0x3Fu) << 12) | ((b2 & 0x3Fu) << 6) | (b3 & 0x3Fu);
        if (v < 0x10000 || v > 0x10FFFF) return 0;
        w = 4;
    } else return 0;
    if (a.raw_docmask)
        for (int k = 1; k < w; ++k) if (raw_docstart(a, q + k)) return 0;
    *cp = v;
    return w;
}

GTOK_DEV bool nfc_attention(const DeviceTables& tb, uint32_t cp) {
    if (cp < 0x300) return false;
    if (cp < 0x10000) return (ldg(tb.nfc_attn_bits + (cp >> 5)) >> (cp & 31)) & 1u;
    uint32_t lo = 0, hi = tb.nfc_attn_sup_n;            // first range with lo > cp
    while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (ldg(tb.nfc_attn_sup + 2 * mid) <= cp) lo = mid + 1; else hi = mid; }
    return lo > 0 && cp <= ldg(tb.nfc_attn_sup + 2 * (lo - 1) + 1);
}

// Combining class (low byte) and index + 1 into nfc_decomp (from bit 8) of cp, 0 for a codepoint that has
// neither: one hashed look-up (a binary search of each list was ten dependent loads per codepoint of a stretch).
GTOK_DEV uint32_t nfc_cp_info(const DeviceTables& tb, uint32_t cp) {
    for (uint32_t at = nfc_cp_hash(cp) & tb.nfc_cp_hash_mask;; at = (at + 1) & tb.nfc_cp_hash_mask) {
        const uint32_t k = ldg(tb.nfc_cp_hash + 2 * at);
        if (k == cp) return ldg(tb.nfc_cp_hash + 2 * at + 1);
        if (k == 0xFFFFFFFFu) return 0;
    }
}
GTOK_DEV uint32_t nfc_ccc(const DeviceTables& tb, uint32_t cp) {
    if (cp < 0x300) return 0;
    return nfc_cp_info(tb, cp) & 0xFFu;
}

GTOK_DEV uint32_t nfc_compose(const DeviceTables& tb, uint32_t x, uint32_t y) {   // 0 when the pair does not compose
    constexpr uint32_t SB = 0xAC00, LB = 0x1100, VB = 0x1161, TB = 0x11A7, LC = 19, VC = 21, TC = 28;
    if (x >= LB && x < LB + LC && y >= VB && y < VB + VC) return SB + ((x - LB) * VC + (y - VB)) * TC;
    if (x >= SB && x < SB + LC * VC * TC && (x - SB) % TC == 0 && y > TB && y < TB + TC) return x + (y - TB);
    // (hashed: a binary search of the thousand pairs was ten dependent loads, most of a stretch's time)
    for (uint32_t at = nfc_comp_hash(x, y) & tb.nfc_comp_hash_mask;; at = (at + 1) & tb.nfc_comp_hash_mask) {
#if defined(__CUDA_ARCH__)
        const uint4 s = __ldg(reinterpret_cast<const uint4*>(tb.nfc_comp_hash) + at);
        const uint32_t f = s.x, sec = s.y, comp = s.z;
#else
        const uint32_t f = tb.nfc_comp_hash[4 * at], sec = tb.nfc_comp_hash[4 * at + 1], comp = tb.nfc_comp_hash[4 * at + 2];
#endif
        if (f == 0xFFFFFFFFu) break;
        if (f == x && sec == y) return comp;
    }
    return 0;
}

struct NfcBuf {
    uint32_t cp[kNfcMaxCps];
    uint8_t cc[kNfcMaxCps];
    int n;
    bool over;
};

GTOK_DEV void nfc_push1(const DeviceTables& tb, NfcBuf& b, uint32_t cp) {
    if (b.n >= kNfcMaxCps) { b.over = true; return; }
    b.cp[b.n] = cp;
    b.cc[b.n] = static_cast<uint8_t>(nfc_ccc(tb, cp));
    ++b.n;
}
// Appends the full canonical decomposition of cp.
GTOK_DEV void nfc_push(const DeviceTables& tb, NfcBuf& b, uint32_t cp) {
    constexpr uint32_t SB = 0xAC00, LB = 0x1100, VB = 0x1161, TB = 0x11A7, VC = 21, TC = 28, SC = 19 * VC * TC;
    if (cp >= SB && cp < SB + SC) {
        const uint32_t s = cp - SB;
        nfc_push1(tb, b, LB + s / (VC * TC));
        nfc_push1(tb, b, VB + (s % (VC * TC)) / TC);
        if (s % TC) nfc_push1(tb, b, TB + s % TC);
        return;
    }
    if (cp >= 0xC0) {
        const uint32_t info = nfc_cp_info(tb, cp);
        if (info >> 8) {
            const uint32_t lo = (info >> 8) - 1u;
            const uint32_t k = ldg(tb.nfc_decomp + 6 * lo + 1);
            for (uint32_t i = 0; i < k && i < 4; ++i) nfc_push1(tb, b, ldg(tb.nfc_decomp + 6 * lo + 2 + i));
            return;
        }
        if (b.n >= kNfcMaxCps) { b.over = true; return; }
        b.cp[b.n] = cp;
        b.cc[b.n] = static_cast<uint8_t>(info & 0xFFu);
        ++b.n;
        return;
    }
    nfc_push1(tb, b, cp);
}

GTOK_DEV uint32_t utf8_width(uint32_t cp) { return cp < 0x80 ? 1u : cp < 0x800 ? 2u : cp < 0x10000 ? 3u : 4u; }

// NFC of the stretch that begins at a0; p is its first attention codepoint (a0 == p when no
// codepoint precedes the run).  Returns the length in bytes of the result and, when `out` is
// given, writes it at out[at...] as far as it fits below `cap`.
GTOK_DEV_NOINLINE uint32_t nfc_stretch(const EncodeArgs& a, uint32_t a0, uint32_t p, uint32_t n, uint8_t* out, uint32_t at, uint32_t cap) {
    uint32_t cp = 0;
    // By far the most common stretch, decided without the general machinery: an ASCII character,
    // one combining mark of U+0300..U+036F that has no decomposition of its own, then something
    // that needs no attention.  The pair either composes or stays as it is.
    if (a0 + 1 == p) {
        const int w1 = nfc_decode(a, p, n, &cp);
        if (w1 == 2 && cp >= 0x300 && cp <= 0x36F && cp != 0x340 && cp != 0x341 && cp != 0x343 && cp != 0x344) {
            const uint32_t q = p + 2;
            uint32_t nx = 0;
            const bool ends = q >= n || raw_docstart(a, q) || nfc_decode(a, q, n, &nx) == 0 || !nfc_attention(a.tb, nx);
            if (ends) {
                const uint32_t b0 = ldg(a.raw + a0);
                const uint32_t m = nfc_compose(a.tb, b0, cp);
                const uint32_t len = m ? utf8_width(m) : 3u;
                if (out && at + len <= cap) {
                    uint8_t* o = out + at;
                    if (!m) { o[0] = static_cast<uint8_t>(b0); o[1] = static_cast<uint8_t>(0xC0 | (cp >> 6)); o[2] = static_cast<uint8_t>(0x80 | (cp & 0x3F)); }
                    else if (len == 2) { o[0] = static_cast<uint8_t>(0xC0 | (m >> 6)); o[1] = static_cast<uint8_t>(0x80 | (m & 0x3F)); }
                    else { o[0] = static_cast<uint8_t>(0xE0 | (m >> 12)); o[1] = static_cast<uint8_t>(0x80 | ((m >> 6) & 0x3F)); o[2] = static_cast<uint8_t>(0x80 | (m & 0x3F)); }
                }
                return len;
            }
        }
    }
    NfcBuf b;
    b.n = 0;
    b.over = false;
    if (a0 < p) { nfc_decode(a, a0, n, &cp); nfc_push(a.tb, b, cp); }
    for (uint32_t q = p; q < n;) {
        const int w = nfc_decode(a, q, n, &cp);
        if (w == 0) break;
        if (q > p && (!nfc_attention(a.tb, cp) || raw_docstart(a, q))) break;
        nfc_push(a.tb, b, cp);
        if (b.over) break;
        q += w;
    }
    if (b.over) { global_or(a.ctl + CTL_ERR, kErrNfcLong); return 0; }
    // canonical order: a stable sort of every run of non-starters by combining class
    for (int i = 1; i < b.n; ++i) {
        const uint32_t kc = b.cc[i], kp = b.cp[i];
        if (kc == 0) continue;
        int j = i;
        while (j > 0 && b.cc[j - 1] != 0 && b.cc[j - 1] > kc) { b.cp[j] = b.cp[j - 1]; b.cc[j] = b.cc[j - 1]; --j; }
        b.cp[j] = kp;
        b.cc[j] = static_cast<uint8_t>(kc);
    }
    // canonical composition, in place
    int m = 0, starter = -1;
    uint32_t last_cc = 0;
    for (int i = 0; i < b.n; ++i) {
        const uint32_t c = b.cc[i], x = b.cp[i];
        if (starter >= 0) {
            const bool adjacent = m == starter + 1;
            if (adjacent || (last_cc != 0 && last_cc < c)) {
                const uint32_t comp = nfc_compose(a.tb, b.cp[starter], x);
                if (comp) { b.cp[starter] = comp; continue; }
            }
        }
        if (c == 0) { starter = m; last_cc = 0; } else last_cc = c;
        b.cp[m] = x;
        b.cc[m] = static_cast<uint8_t>(c);
        ++m;
    }
    uint32_t len = 0;
    for (int i = 0; i < m; ++i) {
        const uint32_t x = b.cp[i], w = utf8_width(x);
        if (out && at + len + w <= cap) {
            uint8_t* o = out + at + len;
            if (w == 1) o[0] = static_cast<uint8_t>(x);
            else if (w == 2) { o[0] = static_cast<uint8_t>(0xC0 | (x >> 6)); o[1] = static_cast<uint8_t>(0x80 | (x & 0x3F)); }
            else if (w == 3) {
                o[0] = static_cast<uint8_t>(0xE0 | (x >> 12)); o[1] = static_cast<uint8_t>(0x80 | ((x >> 6) & 0x3F));
                o[2] = static_cast<uint8_t>(0x80 | (x & 0x3F));
            } else {
                o[0] = static_cast<uint8_t>(0xF0 | (x >> 18)); o[1] = static_cast<uint8_t>(0x80 | ((x >> 12) & 0x3F));
                o[2] = static_cast<uint8_t>(0x80 | ((x >> 6) & 0x3F)); o[3] = static_cast<uint8_t>(0x80 | (x & 0x3F));
            }
        }
        len += w;
    }
    return len;
}

// The 16 bytes at c0 (a multiple of 16) as four little-endian words.
GTOK_DEV void load16(const uint8_t* p, uint32_t w[4]) {
#if defined(__CUDA_ARCH__)
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
#else
    for (int k = 0; k < 4; ++k) w[k] = static_cast<uint32_t>(p[4 * k]) | (static_cast<uint32_t>(p[4 * k + 1]) << 8) |
                                       (static_cast<uint32_t>(p[4 * k + 2]) << 16) | (static_cast<uint32_t>(p[4 * k + 3]) << 24);
#endif
}
// High bit of every byte of w that is 0xCC or above (only such bytes can lead an attention codepoint).
GTOK_DEV uint32_t cand_bytes(uint32_t w) { return w & ((w & 0x7F7F7F7Fu) + 0x34343434u) & 0x80808080u; }

// Attention masks of the 16-byte chunk at c0: bit i of *lead = an attention codepoint begins
// at c0 + i, bit i of *fill = byte c0 + i belongs to one.
GTOK_DEV void nfc_chunk_masks(const EncodeArgs& a, long long c0s, uint32_t n, uint32_t* lead, uint32_t* fill) {
    *lead = 0;
    *fill = 0;
    if (c0s < 0 || c0s >= static_cast<long long>(n)) return;
    const uint32_t c0 = static_cast<uint32_t>(c0s);
    uint32_t w[4];
    load16(a.raw + c0, w);
    uint32_t before = 0;                                   // bytes c0-4 .. c0-1
    if (c0) {
        const uint8_t* q = a.raw + c0 - 4;
        before = static_cast<uint32_t>(ldg(q)) | (static_cast<uint32_t>(ldg(q + 1)) << 8) | (static_cast<uint32_t>(ldg(q + 2)) << 16) |
                 (static_cast<uint32_t>(ldg(q + 3)) << 24);
        before &= 0xFFFFFF00u;                             // a codepoint that begins 4 bytes back cannot reach the chunk
    }
    const uint32_t c[5] = {cand_bytes(before), cand_bytes(w[0]), cand_bytes(w[1]), cand_bytes(w[2]), cand_bytes(w[3])};
    if ((c[0] | c[1] | c[2] | c[3] | c[4]) == 0) return;
    uint32_t l = 0, f = 0;
    for (int k = 0; k < 5; ++k) {
        uint32_t m = c[k];
        while (m) {
            const int bit = ffs32(m);
            m &= m - 1;
            const int i = 4 * (k - 1) + (bit >> 3);        // byte offset from c0, -3 .. 15
            const uint32_t word = k == 0 ? before : w[k - 1];
            const uint32_t b = (word >> (bit - 7)) & 0xFFu;
            if (b > 0xF4 || ((a.tb.nfc_lead_quiet[b >> 5] >> (b & 31)) & 1u)) continue;   // no attention codepoint begins with this byte
            const uint32_t pos = c0 + i;                   // i >= -3 and c0 >= 16 whenever i < 0
            if (pos >= n) continue;
            uint32_t cp;
            const int wd = nfc_decode(a, pos, n, &cp);
            if (wd == 0 || !nfc_attention(a.tb, cp)) continue;
            if (i >= 0) l |= 1u << i;
            for (int t = 0; t < wd; ++t) if (i + t >= 0 && i + t < 16) f |= 1u << (i + t);
        }
    }
    *lead = l;
    *fill = f;
}

template <class Blk>
GTOK_DEV void nfc_tile(Blk& blk, const EncodeArgs& a, NfcSmem& sm, int tile) {
    const uint32_t n = ldg(a.raw_meta);
    const uint32_t n_docs = ldg(a.raw_meta + 1);
    const bool plain = ldg(a.raw_meta + 2) != 0;
    const uint32_t t0 = static_cast<uint32_t>(tile) * kTile;
    const uint32_t n_tiles = (n + kTile - 1) / kTile;
    const uint32_t cap = a.text_cap;
    auto mark = [&](int slot) {
        if (!a.phase_clk) return;
        blk.par([&](int tid) {
            if (tid != 0) return;
            unsigned long long t = cycle_now();
            if (slot >= 0) add_cycles(a.phase_clk + slot, t - sm.clk_last);
            sm.clk_last = t;
        });
    };
    mark(-1);
    // ---- N1: attention masks per chunk ----
    blk.par([&](int tid) {
        uint32_t l = 0, f = 0;
        if (!plain) nfc_chunk_masks(a, static_cast<long long>(t0) + tid * kPer, n, &l, &f);
        sm.attl[tid + 1] = static_cast<uint16_t>(l);
        sm.attf[tid + 1] = static_cast<uint16_t>(f);
        if (tid < 2) {                                     // the chunk before the tile and the one after it
            l = f = 0;
            const long long c0 = tid == 0 ? static_cast<long long>(t0) - kPer : static_cast<long long>(t0) + kTile;
            if (!plain) nfc_chunk_masks(a, c0, n, &l, &f);
            sm.attl[tid == 0 ? 0 : kThreads + 1] = static_cast<uint16_t>(l);
            sm.attf[tid == 0 ? 0 : kThreads + 1] = static_cast<uint16_t>(f);
        }
    });
    mark(27);
    // ---- N2: stretches; bytes each thread will emit ----
    blk.par([&](int tid) {
        const uint32_t c0 = t0 + tid * kPer;
        uint32_t valid = 0;
        if (c0 < n) valid = n - c0 >= static_cast<uint32_t>(kPer) ? 0xFFFFu : ((1u << (n - c0)) - 1u);
        // bit 16 + i of the windows stands for byte c0 + i
        const unsigned long long wl = static_cast<unsigned long long>(sm.attl[tid]) | (static_cast<unsigned long long>(sm.attl[tid + 1]) << 16) |
                                      (static_cast<unsigned long long>(sm.attl[tid + 2]) << 32);
        const unsigned long long wf = static_cast<unsigned long long>(sm.attf[tid]) | (static_cast<unsigned long long>(sm.attf[tid + 1]) << 16) |
                                      (static_cast<unsigned long long>(sm.attf[tid + 2]) << 32);
        uint32_t drop = sm.attf[tid + 1], own = 0, extra = 0, kept = 0;
        // run starts at c0 .. c0 + 19: the codepoint before such a run may lie in this chunk
        unsigned long long rs = wl & ~(wf << 1);
        if (a.raw_docmask && (wl >> 16)) {
            unsigned long long dm = 0;
            for (int i = 0; i < 20; ++i) if (((wl >> (16 + i)) & 1ull) && c0 + i < n && raw_docstart(a, c0 + i)) dm |= 1ull << (16 + i);
            rs |= dm;
        }
        rs = (rs >> 16) & 0xFFFFFull;
        while (rs) {
            int i = 0;
            while (!((rs >> i) & 1ull)) ++i;
            rs &= rs - 1;
            const uint32_t p = c0 + i;
            if (p >= n) break;
            uint32_t a0 = p;
            if (p > 0 && !raw_docstart(a, p)) {
                uint32_t q = p - 1;
                int steps = 0;
                while (q > 0 && steps < 3 && (ldg(a.raw + q) & 0xC0) == 0x80) { --q; ++steps; }
                uint32_t cp;
                const int w = nfc_decode(a, q, n, &cp);
                if (w != 0 && q + w == p) a0 = q;
            }
            for (uint32_t t = a0; t < p; ++t) if (t >= c0 && t < c0 + kPer) drop |= 1u << (t - c0);
            if (a0 >= c0 && a0 < c0 + kPer) {
                own |= 1u << (a0 - c0);
                drop |= 1u << (a0 - c0);
                // (the first one's bytes are kept for the write phase when they fit: working a stretch out is one thread's
                // job while its warp waits, and most of what this kernel costs)
                const bool keep = own == (1u << (a0 - c0));
                const uint32_t len = nfc_stretch(a, a0, p, n, keep ? sm.sres[tid] : nullptr, 0, keep ? 12u : 0u);
                kept = keep && len <= 12u ? len : 0u;
                extra += len;
            }
        }
        sm.slen[tid] = static_cast<uint8_t>(popc32(own) == 1 ? kept : 0u);
        sm.drop[tid] = static_cast<uint16_t>(drop);
        sm.own[tid] = static_cast<uint16_t>(own);
        sm.scan[tid] = static_cast<uint32_t>(popc32(valid & ~drop)) + extra;
    });
    uint32_t total = 0;
    blk.excl_scan(sm.scan, &total);
    mark(24);
    // ---- N3: the tile's place in the output ----
    const uint32_t base = blk.lookback(a.st0, tile, total, a.ctl);
    mark(25);
    // ---- N4: write ----
    // Once a document has changed length its bytes no longer land on the 16-byte lines they came from.  The
    // tile's output is therefore put together in shared memory, shifted so that shared-memory lines are
    // output lines, and goes out line by line (the ragged first and last line byte by byte: the neighbouring
    // tiles write the rest of those).  A tile that grows beyond the buffer writes its bytes one by one.
    const uint32_t shift = base & 15u;
    const bool staged = shift + total <= static_cast<uint32_t>(kNfcStage);
    blk.par([&](int tid) {
        const uint32_t c0 = t0 + tid * kPer;
        if (c0 >= n) return;
        uint32_t at = base + sm.scan[tid];
        const uint32_t drop = sm.drop[tid], own = sm.own[tid];
        const uint32_t cnt = n - c0 >= static_cast<uint32_t>(kPer) ? kPer : n - c0;
        uint32_t docbits = 0;
        if (a.raw_docmask) docbits = (ldg(a.raw_docmask + (c0 >> 5)) >> (c0 & 31)) & 0xFFFFu;
        uint32_t w[4];
        load16(a.raw + c0, w);
        if (staged) {
            // same walk as below, into the buffer: position `at` of the output is byte at - base + shift there
            uint32_t la = shift + sm.scan[tid];
            if (drop == 0 && docbits == 0 && cnt == kPer) {
                if ((la & 3u) == 0) { uint32_t* d = reinterpret_cast<uint32_t*>(sm.outb + la); d[0] = w[0]; d[1] = w[1]; d[2] = w[2]; d[3] = w[3]; }
                else for (int i = 0; i < kPer; ++i) sm.outb[la + i] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
                return;
            }
            for (uint32_t i = 0; i < cnt; ++i) {
                if ((docbits >> i) & 1u) {
                    const uint32_t r = c0 + i;
                    uint32_t lo = 0, hi = n_docs + 1;
                    while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (ldg(a.raw_doc_off + mid) < r) lo = mid + 1; else hi = mid; }
                    for (uint32_t d = lo; d <= n_docs && ldg(a.raw_doc_off + d) == r; ++d) a.norm_doc_off[d] = base + (la - shift);
                }
                if ((own >> i) & 1u) {
                    const uint32_t a0 = c0 + i;
                    uint32_t p = a0;
                    if (!((sm.attl[tid + 1] >> i) & 1u)) {
                        uint32_t cp;
                        p = a0 + static_cast<uint32_t>(nfc_decode(a, a0, n, &cp));
                    }
                    const uint32_t kept = sm.slen[tid];
                    if (kept) { for (uint32_t t = 0; t < kept; ++t) sm.outb[la + t] = sm.sres[tid][t]; la += kept; }
                    else la += nfc_stretch(a, a0, p, n, sm.outb, la, kNfcStage);
                } else if (!((drop >> i) & 1u)) {
                    sm.outb[la] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
                    ++la;
                }
            }
            return;
        }
        if (drop == 0 && docbits == 0 && cnt == kPer && (at & 15u) == 0 && at + kPer <= cap) {
#if defined(__CUDA_ARCH__)
            *reinterpret_cast<uint4*>(a.norm_text + at) = make_uint4(w[0], w[1], w[2], w[3]);
#else
            for (int i = 0; i < kPer; ++i) a.norm_text[at + i] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
#endif
            return;
        }
        for (uint32_t i = 0; i < cnt; ++i) {
            if ((docbits >> i) & 1u) {
                // every document that begins at this byte begins at `at` in the output
                const uint32_t r = c0 + i;
                uint32_t lo = 0, hi = n_docs + 1;
                while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (ldg(a.raw_doc_off + mid) < r) lo = mid + 1; else hi = mid; }
                for (uint32_t d = lo; d <= n_docs && ldg(a.raw_doc_off + d) == r; ++d) a.norm_doc_off[d] = at;
            }
            if ((own >> i) & 1u) {
                const uint32_t a0 = c0 + i;
                uint32_t p = a0;
                if (!((sm.attl[tid + 1] >> i) & 1u)) {
                    uint32_t cp;
                    p = a0 + static_cast<uint32_t>(nfc_decode(a, a0, n, &cp));
                }
                at += nfc_stretch(a, a0, p, n, a.norm_text, at, cap);
            } else if (!((drop >> i) & 1u)) {
                if (at < cap) a.norm_text[at] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
                ++at;
            }
        }
    });
    mark(28);
    if (staged && total) {
        blk.par([&](int tid) {
            const uint32_t line0 = base - shift, lines = (shift + total + 15u) / 16u;
            for (uint32_t l = tid; l < lines; l += kThreads) {
                const uint32_t lo_b = l == 0 ? shift : 0u;                                      // first and one-past-last byte of the line that are this tile's
                const uint32_t hi_b = (l + 1) * 16u <= shift + total ? 16u : shift + total - l * 16u;
                const uint32_t g0 = line0 + l * 16u;
                if (lo_b == 0 && hi_b == 16u && g0 + 16u <= cap) {
#if defined(__CUDA_ARCH__)
                    *reinterpret_cast<uint4*>(a.norm_text + g0) = *reinterpret_cast<const uint4*>(sm.outb + l * 16u);
#else
                    for (int i = 0; i < 16; ++i) a.norm_text[g0 + i] = sm.outb[l * 16u + i];
#endif
                    continue;
                }
                for (uint32_t i = lo_b; i < hi_b; ++i) if (g0 + i < cap) a.norm_text[g0 + i] = sm.outb[l * 16u + i];
            }
        });
    }
    if (static_cast<uint32_t>(tile) + 1 == n_tiles) {
        blk.par([&](int tid) {
            const uint32_t new_n = base + total;
            if (a.raw_doc_off) {
                // documents that begin at the end of the text (empty trailing documents, the closing offset)
                uint32_t lo = 0, hi = n_docs + 1;
                while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (ldg(a.raw_doc_off + mid) < n) lo = mid + 1; else hi = mid; }
                for (uint32_t d = lo + tid; d <= n_docs; d += kThreads) a.norm_doc_off[d] = new_n;
            }
            if (tid != 0) return;
            const bool fits = new_n <= cap;
            if (!fits) global_or(a.ctl + CTL_ERR, kErrNfcFull);
            a.norm_meta[0] = fits ? new_n : 0u;
            a.norm_meta[1] = n_docs;
            a.status[2] = new_n;
        });
    }
    mark(26);
}

}  // namespace gtok
