// Partitioning of one encode job over the GPUs of a box.  Pure host code.
//
// Documents of a batch are independent, so a batch is cut into contiguous
// document ranges of about equal byte count.  One long document is cut only at
// positions where a pre-token provably starts whatever precedes it and no
// run-level rule can reach across: an ASCII letter, then a single 0x20 space,
// then an ASCII letter, with the cut in front of the space.  For all four
// families the space opens the next word's pre-token there (" word"), a regular
// expression never looks behind its match start, and cutting the text in front
// of the space ends the left part on a letter run exactly as the space would; the
// three bytes are inert under NFC and cannot lie inside an added-token literal
// unless a literal contains that very pattern, which is checked.  Each part is
// then an ordinary document, so concatenating the parts' ids gives the ids of
// the whole text.  The only data that crosses GPUs is the parts' token counts.
#pragma once
#include <cstdint>
#include <string>
#include <algorithm>
#include <vector>

#include "vocab_host.h"

namespace gtok {

inline bool ascii_letter(uint8_t b) { return (b >= 'a' && b <= 'z') || (b >= 'A' && b <= 'Z'); }

// True when position p (in front of text[p]) is a safe cut.
inline bool safe_cut(const HostVocab& hv, const uint8_t* text, uint64_t len, uint64_t p) {
    if (p == 0 || p + 1 >= len) return false;
    if (!(ascii_letter(text[p - 1]) && text[p] == 0x20 && ascii_letter(text[p + 1]))) return false;
    // (Gemma-3 shape: the space is the character U+2581 of a model that merges across everything; the cut holds
    // when no rule can join the letter before it to a U+2581 after it and the vocabulary has that letter)
    if (hv.family == Family::Gemma3) {
        if (std::binary_search(hv.sp_before_bar.begin(), hv.sp_before_bar.end(), static_cast<uint32_t>(text[p - 1]))) return false;
        auto it = std::lower_bound(hv.sp_chars.begin(), hv.sp_chars.end(), std::make_pair(static_cast<uint32_t>(text[p - 1]), 0u));
        if (it == hv.sp_chars.end() || it->first != text[p - 1]) return true;      // a byte on its own: a cut on either side of it
    }
    // No added-token literal occurrence may overlap the three bytes.
    if (hv.added_max_bytes) {
        uint64_t lo = p + 2 > hv.added_max_bytes ? p + 2 - hv.added_max_bytes : 0;
        for (uint64_t s = lo; s <= p + 1; ++s) {
            for (const AddedToken& a : hv.added) {
                const std::string& c = a.content;
                if (s + c.size() > len || s + c.size() + 1 <= p) continue;     // ends before text[p-1]
                if (std::char_traits<char>::compare(reinterpret_cast<const char*>(text + s), c.data(), c.size()) == 0) return false;
            }
        }
    }
    return true;
}

// Cuts `text` into n_parts pieces of about equal size at safe positions.
// out[0] = 0, out[n_parts] = len; a piece may be empty when no safe cut exists
// between the previous cut and the end.
inline void plan_chunks(const HostVocab& hv, const uint8_t* text, uint64_t len, uint32_t n_parts, std::vector<uint64_t>& out) {
    out.assign(n_parts + 1, len);
    out[0] = 0;
    uint64_t prev = 0;
    for (uint32_t k = 1; k < n_parts; ++k) {
        uint64_t want = len * k / n_parts;
        if (want < prev) want = prev;
        uint64_t p = want;
        while (p < len && !safe_cut(hv, text, len, p)) ++p;
        if (p >= len) p = len;
        out[k] = p;
        prev = p;
    }
}

// Cuts n_docs documents (n_docs + 1 ascending byte offsets) into n_parts contiguous
// ranges of about equal byte count.  out has n_parts + 1 document indices.
inline void plan_documents(const uint32_t* doc_off, uint32_t n_docs, uint32_t n_parts, std::vector<uint32_t>& out) {
    out.assign(n_parts + 1, n_docs);
    out[0] = 0;
    const uint64_t total = static_cast<uint64_t>(doc_off[n_docs]) - doc_off[0];
    uint32_t d = 0;
    for (uint32_t k = 1; k < n_parts; ++k) {
        uint64_t want = doc_off[0] + total * k / n_parts;
        while (d < n_docs && doc_off[d] < want) ++d;
        out[k] = d;
    }
}

}  // namespace gtok
