// See nfc_host.h.
#include "nfc_host.h"

#include <algorithm>
#include <vector>

#include "device_tables.h"
#include "nfc_tables.h"

namespace gtok {

namespace {

constexpr uint32_t kSBase = 0xAC00, kLBase = 0x1100, kVBase = 0x1161, kTBase = 0x11A7;
constexpr uint32_t kLCount = 19, kVCount = 21, kTCount = 28, kNCount = kVCount * kTCount, kSCount = kLCount * kNCount;

uint32_t ccc_of(uint32_t cp) {
    if (cp < 0x300) return 0;
    const GtokNfcCcc* e = std::lower_bound(gtok_nfc_ccc, gtok_nfc_ccc + GTOK_NFC_CCC_LEN, cp,
                                           [](const GtokNfcCcc& x, uint32_t v) { return x.cp < v; });
    return (e != gtok_nfc_ccc + GTOK_NFC_CCC_LEN && e->cp == cp) ? e->ccc : 0;
}
// One bit per BMP codepoint, set for the codepoints that need attention.
struct AttnBits {
    uint64_t w[1024];
    AttnBits() {
        for (uint64_t& x : w) x = 0;
        for (uint32_t r = 0; r < GTOK_NFC_ATTN_LEN; ++r)
            for (uint32_t cp = gtok_nfc_attn[r].lo; cp <= gtok_nfc_attn[r].hi && cp < 0x10000; ++cp) w[cp >> 6] |= 1ull << (cp & 63);
    }
};
bool needs_attention(uint32_t cp) {
    if (cp < 0x300) return false;
    static const AttnBits bits;
    if (cp < 0x10000) return (bits.w[cp >> 6] >> (cp & 63)) & 1u;
    const GtokNfcRange* e = std::upper_bound(gtok_nfc_attn, gtok_nfc_attn + GTOK_NFC_ATTN_LEN, cp,
                                             [](uint32_t v, const GtokNfcRange& r) { return v < r.lo; });
    return e != gtok_nfc_attn && cp <= (e - 1)->hi;
}
void decompose(uint32_t cp, std::vector<uint32_t>& out) {
    if (cp >= kSBase && cp < kSBase + kSCount) {
        uint32_t s = cp - kSBase;
        out.push_back(kLBase + s / kNCount);
        out.push_back(kVBase + (s % kNCount) / kTCount);
        if (s % kTCount) out.push_back(kTBase + s % kTCount);
        return;
    }
    if (cp >= 0xC0) {
        const GtokNfcDecomp* e = std::lower_bound(gtok_nfc_decomp, gtok_nfc_decomp + GTOK_NFC_DECOMP_LEN, cp,
                                                  [](const GtokNfcDecomp& x, uint32_t v) { return x.cp < v; });
        if (e != gtok_nfc_decomp + GTOK_NFC_DECOMP_LEN && e->cp == cp) {
            for (uint32_t i = 0; i < e->n; ++i) out.push_back(e->d[i]);
            return;
        }
    }
    out.push_back(cp);
}
uint32_t compose(uint32_t a, uint32_t b) {   // 0 when the pair does not compose
    if (a >= kLBase && a < kLBase + kLCount && b >= kVBase && b < kVBase + kVCount)
        return kSBase + ((a - kLBase) * kVCount + (b - kVBase)) * kTCount;
    if (a >= kSBase && a < kSBase + kSCount && (a - kSBase) % kTCount == 0 && b > kTBase && b < kTBase + kTCount)
        return a + (b - kTBase);
    const GtokNfcComp* e = std::lower_bound(gtok_nfc_comp, gtok_nfc_comp + GTOK_NFC_COMP_LEN, std::make_pair(a, b),
                                            [](const GtokNfcComp& x, const std::pair<uint32_t, uint32_t>& v) {
                                                return x.first != v.first ? x.first < v.first : x.second < v.second;
                                            });
    return (e != gtok_nfc_comp + GTOK_NFC_COMP_LEN && e->first == a && e->second == b) ? e->composite : 0;
}

// Strict UTF-8 decode at p (n bytes available): width, or 0 when the bytes are not a
// well-formed sequence (overlong, surrogate, out of range, truncated).
int decode(const uint8_t* p, size_t n, uint32_t* cp) {
    uint8_t b = p[0];
    if (b < 0x80) { *cp = b; return 1; }
    if (b >= 0xC2 && b <= 0xDF && n >= 2 && (p[1] & 0xC0) == 0x80) { *cp = ((b & 0x1Fu) << 6) | (p[1] & 0x3Fu); return 2; }
    if ((b & 0xF0) == 0xE0 && n >= 3 && (p[1] & 0xC0) == 0x80 && (p[2] & 0xC0) == 0x80) {
        uint32_t v = ((b & 0x0Fu) << 12) | ((p[1] & 0x3Fu) << 6) | (p[2] & 0x3Fu);
        if (v < 0x800 || (v >= 0xD800 && v <= 0xDFFF)) return 0;
        *cp = v;
        return 3;
    }
    if (b >= 0xF0 && b <= 0xF4 && n >= 4 && (p[1] & 0xC0) == 0x80 && (p[2] & 0xC0) == 0x80 && (p[3] & 0xC0) == 0x80) {
        uint32_t v = ((b & 0x07u) << 18) | ((p[1] & 0x3Fu) << 12) | ((p[2] & 0x3Fu) << 6) | (p[3] & 0x3Fu);
        if (v < 0x10000 || v > 0x10FFFF) return 0;
        *cp = v;
        return 4;
    }
    return 0;
}
void encode(uint32_t cp, std::string& s) {
    if (cp < 0x80) s.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { s.push_back(static_cast<char>(0xC0 | (cp >> 6))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
        s.push_back(static_cast<char>(0xE0 | (cp >> 12))); s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
        s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
        s.push_back(static_cast<char>(0xF0 | (cp >> 18))); s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
        s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
}

// NFC of one stretch of codepoints, in place.
void normalize_stretch(std::vector<uint32_t>& cps, std::vector<uint32_t>& tmp) {
    tmp.clear();
    for (uint32_t cp : cps) decompose(cp, tmp);
    // canonical ordering: stable sort of each run of non-starters by combining class
    for (size_t i = 0; i < tmp.size();) {
        if (ccc_of(tmp[i]) == 0) { ++i; continue; }
        size_t j = i;
        while (j < tmp.size() && ccc_of(tmp[j]) != 0) ++j;
        std::stable_sort(tmp.begin() + i, tmp.begin() + j, [](uint32_t x, uint32_t y) { return ccc_of(x) < ccc_of(y); });
        i = j;
    }
    // canonical composition
    cps.clear();
    size_t starter = SIZE_MAX;
    uint32_t last_ccc = 0;
    for (uint32_t cp : tmp) {
        const uint32_t c = ccc_of(cp);
        if (starter != SIZE_MAX) {
            const bool adjacent = cps.size() == starter + 1;
            if (adjacent || (last_ccc != 0 && last_ccc < c)) {
                uint32_t m = compose(cps[starter], cp);
                if (m) { cps[starter] = m; continue; }
            }
        }
        if (c == 0) { starter = cps.size(); last_ccc = 0; }
        else last_ccc = c;
        cps.push_back(cp);
    }
}

}  // namespace

void nfc_table_words(NfcWords& out) {
    out.attn_bits.assign(2048, 0);
    out.attn_sup.clear();
    for (uint32_t r = 0; r < GTOK_NFC_ATTN_LEN; ++r) {
        for (uint32_t cp = gtok_nfc_attn[r].lo; cp <= gtok_nfc_attn[r].hi && cp < 0x10000; ++cp) out.attn_bits[cp >> 5] |= 1u << (cp & 31);
        if (gtok_nfc_attn[r].hi >= 0x10000) {
            out.attn_sup.push_back(gtok_nfc_attn[r].lo < 0x10000 ? 0x10000 : gtok_nfc_attn[r].lo);
            out.attn_sup.push_back(gtok_nfc_attn[r].hi);
        }
    }
    // lead bytes under which no such codepoint lies (all of Cyrillic's D0 and D1, the CJK ideographs' E4..E9, ...)
    for (uint32_t& w : out.lead_quiet) w = 0xFFFFFFFFu;
    for (uint32_t r = 0; r < GTOK_NFC_ATTN_LEN; ++r)
        for (uint32_t cp = gtok_nfc_attn[r].lo; cp <= gtok_nfc_attn[r].hi; ++cp) {
            const uint32_t lead = cp < 0x80 ? cp : cp < 0x800 ? 0xC0u | (cp >> 6) : cp < 0x10000 ? 0xE0u | (cp >> 12) : 0xF0u | (cp >> 18);
            out.lead_quiet[lead >> 5] &= ~(1u << (lead & 31));
        }
    out.ccc.clear();
    for (uint32_t i = 0; i < GTOK_NFC_CCC_LEN; ++i) { out.ccc.push_back(gtok_nfc_ccc[i].cp); out.ccc.push_back(gtok_nfc_ccc[i].ccc); }
    out.decomp.clear();
    for (uint32_t i = 0; i < GTOK_NFC_DECOMP_LEN; ++i) {
        out.decomp.push_back(gtok_nfc_decomp[i].cp);
        out.decomp.push_back(gtok_nfc_decomp[i].n);
        for (int k = 0; k < 4; ++k) out.decomp.push_back(gtok_nfc_decomp[i].d[k]);
    }
    out.comp.clear();
    for (uint32_t i = 0; i < GTOK_NFC_COMP_LEN; ++i) {
        out.comp.push_back(gtok_nfc_comp[i].first); out.comp.push_back(gtok_nfc_comp[i].second); out.comp.push_back(gtok_nfc_comp[i].composite);
    }
    {
        // combining class and decomposition of a codepoint behind one hashed look-up (a codepoint in neither list has no slot)
        uint32_t n_slots = 1024;
        while (n_slots < 4 * (GTOK_NFC_CCC_LEN + GTOK_NFC_DECOMP_LEN)) n_slots <<= 1;
        out.cp_hash.assign(static_cast<size_t>(n_slots) * 2, 0xFFFFFFFFu);
        auto slot_of = [&](uint32_t cp) -> uint32_t {
            uint32_t at = nfc_cp_hash(cp) & (n_slots - 1);
            while (out.cp_hash[2 * at] != 0xFFFFFFFFu && out.cp_hash[2 * at] != cp) at = (at + 1) & (n_slots - 1);
            if (out.cp_hash[2 * at] == 0xFFFFFFFFu) { out.cp_hash[2 * at] = cp; out.cp_hash[2 * at + 1] = 0; }
            return at;
        };
        for (uint32_t i = 0; i < GTOK_NFC_CCC_LEN; ++i) out.cp_hash[2 * slot_of(gtok_nfc_ccc[i].cp) + 1] |= gtok_nfc_ccc[i].ccc & 0xFFu;
        for (uint32_t i = 0; i < GTOK_NFC_DECOMP_LEN; ++i) out.cp_hash[2 * slot_of(gtok_nfc_decomp[i].cp) + 1] |= (i + 1) << 8;
    }
    uint32_t slots = 1024;
    while (slots < 4 * GTOK_NFC_COMP_LEN) slots <<= 1;
    out.comp_hash.assign(static_cast<size_t>(slots) * 4, 0xFFFFFFFFu);
    for (uint32_t i = 0; i < GTOK_NFC_COMP_LEN; ++i) {
        uint32_t at = nfc_comp_hash(gtok_nfc_comp[i].first, gtok_nfc_comp[i].second) & (slots - 1);
        while (out.comp_hash[4 * at] != 0xFFFFFFFFu) at = (at + 1) & (slots - 1);
        out.comp_hash[4 * at] = gtok_nfc_comp[i].first; out.comp_hash[4 * at + 1] = gtok_nfc_comp[i].second;
        out.comp_hash[4 * at + 2] = gtok_nfc_comp[i].composite; out.comp_hash[4 * at + 3] = 0;
    }
}

bool nfc_normalize(const uint8_t* text, size_t len, std::string& out) {
    // Every codepoint that can make a text non-NFC is U+0300 or above: lead byte >= 0xCC.
    size_t i = 0;
    bool changed = false;
    size_t copied = 0;                       // text[0, copied) is already in `out` (once anything changed)
    std::vector<uint32_t> cps, tmp;
    std::string piece;
    while (i < len) {
        if (text[i] < 0xCC) {
            // eight ASCII bytes at a time
            while (i + 8 <= len) {
                uint64_t w8;
                __builtin_memcpy(&w8, text + i, 8);
                if (w8 & 0x8080808080808080ull) break;
                i += 8;
            }
            if (i < len && text[i] < 0xCC) ++i;
            continue;
        }
        uint32_t cp;
        int w = decode(text + i, len - i, &cp);
        if (w == 0 || !needs_attention(cp)) { i += w ? w : 1; continue; }
        // By far the most common case, decided without building a stretch: an ASCII character,
        // one combining mark of U+0300..U+036F that has no decomposition of its own, then
        // something that needs no attention.  The pair either composes or stays as it is.
        if (cp <= 0x36F && cp != 0x340 && cp != 0x341 && cp != 0x343 && cp != 0x344 && i > copied && text[i - 1] < 0x80) {
            uint32_t nx = 0;
            int nw = i + w < len ? decode(text + i + w, len - i - w, &nx) : 1;
            if (i + w >= len || (nw != 0 && !needs_attention(nx)) || (nw == 0)) {
                uint32_t m = compose(text[i - 1], cp);
                if (m) {
                    if (!changed) { out.clear(); changed = true; }
                    out.append(reinterpret_cast<const char*>(text + copied), i - 1 - copied);
                    encode(m, out);
                    copied = i + w;
                }
                i += w;
                continue;
            }
        }
        // Stretch: back to the nearest codepoint that is a starter needing no attention
        // (it may combine with what follows), forward to the next such codepoint.
        size_t a = i;
        while (a > copied) {
            size_t q = a - 1;
            while (q > copied && (text[q] & 0xC0) == 0x80) --q;
            uint32_t pc;
            int pw = decode(text + q, len - q, &pc);
            if (pw == 0 || q + pw != a) break;                   // malformed bytes are a barrier
            a = q;
            if (ccc_of(pc) == 0 && !needs_attention(pc)) break;
        }
        size_t b = i;
        cps.clear();
        {
            size_t q = a;
            while (q < i) { uint32_t c2; int w2 = decode(text + q, len - q, &c2); cps.push_back(c2); q += w2; }
        }
        while (b < len) {
            uint32_t c2;
            int w2 = decode(text + b, len - b, &c2);
            if (w2 == 0) break;
            if (b > i && ccc_of(c2) == 0 && !needs_attention(c2)) break;
            cps.push_back(c2);
            b += w2;
        }
        normalize_stretch(cps, tmp);
        piece.clear();
        for (uint32_t c2 : cps) encode(c2, piece);
        if (piece.size() != b - a || piece.compare(0, piece.size(), reinterpret_cast<const char*>(text + a), b - a) != 0) {
            if (!changed) { out.clear(); changed = true; }
            out.append(reinterpret_cast<const char*>(text + copied), a - copied);
            out += piece;
            copied = b;
        }
        i = b;
    }
    if (!changed) return false;
    out.append(reinterpret_cast<const char*>(text + copied), len - copied);
    return true;
}

}  // namespace gtok
