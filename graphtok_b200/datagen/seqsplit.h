// Sequential pre-tokenizer: a direct, cursor-based reading of the three
// pre-tokenizer regular expressions (leftmost match, alternatives tried in
// order, greedy quantifiers with backtracking).  It is deliberately the naive
// formulation: the synthetic-vocabulary trainer uses it to cut its corpus into
// words, and the tests use it as one more independent statement of where
// pre-tokens begin.  Input must be valid UTF-8.
//
//   GPT-2   : 's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//   Llama-3 : (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}|
//             ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//   Qwen2.5 : as Llama-3 with \p{N} in place of \p{N}{1,3}
//   DeepSeek-V3 : three Split steps one after the other, each working on the pieces the one
//             before left (a piece's ends are the text's ends for the next pattern):
//             \p{N}{1,3}   then   [一-龥぀-ゟ゠-ヿ]+   then
//             [!-/:-@\[-`{-~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+|
//              ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//             (matches and the stretches between matches are both pieces)
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../csrc/unicode_class_table.h"
#include "../csrc/unicode_wide_table.h"

namespace gtok_datagen {

enum SplitFamily { kSplitGPT2 = 0, kSplitLlama3 = 1, kSplitQwen25 = 2, kSplitDeepSeek = 3 };

struct Decoded {
    std::vector<uint32_t> cp;     // codepoints
    std::vector<uint32_t> at;     // byte offset of each codepoint, plus the total length
    std::vector<uint8_t> cls;     // 0 L, 1 N, 2 S, 3 other
};

inline void decode_utf8(const uint8_t* s, size_t n, Decoded& d) {
    d.cp.clear(); d.at.clear(); d.cls.clear();
    size_t i = 0;
    while (i < n) {
        uint32_t c = s[i], cp;
        size_t w;
        if (c < 0x80) { cp = c; w = 1; }
        else if ((c & 0xE0) == 0xC0 && i + 1 < n) { cp = ((c & 0x1F) << 6) | (s[i + 1] & 0x3F); w = 2; }
        else if ((c & 0xF0) == 0xE0 && i + 2 < n) { cp = ((c & 0x0F) << 12) | ((s[i + 1] & 0x3F) << 6) | (s[i + 2] & 0x3F); w = 3; }
        else if ((c & 0xF8) == 0xF0 && i + 3 < n) { cp = ((c & 0x07) << 18) | ((s[i + 1] & 0x3F) << 12) | ((s[i + 2] & 0x3F) << 6) | (s[i + 3] & 0x3F); w = 4; }
        else { cp = c; w = 1; }
        d.cp.push_back(cp);
        d.at.push_back(static_cast<uint32_t>(i));
        d.cls.push_back(static_cast<uint8_t>(gtok_uc_lookup(gtok_uc_stage1_init, gtok_uc_stage2_init, cp)));
        i += w;
    }
    d.at.push_back(static_cast<uint32_t>(n));
}

// Length in codepoints of the match at cursor i (always >= 1 for i < n).
inline size_t match_at(const Decoded& d, size_t i, SplitFamily fam) {
    const size_t n = d.cp.size();
    auto C = [&](size_t j) -> int { return j < n ? d.cls[j] : -1; };
    auto P = [&](size_t j) -> uint32_t { return j < n ? d.cp[j] : 0xFFFFFFFFu; };
    const bool ci = fam != kSplitGPT2;
    auto low = [&](uint32_t c) -> uint32_t {
        if (!ci) return c;
        if (c >= 'A' && c <= 'Z') return c + 32;
        if (c == 0x17F) return 's';     // LATIN SMALL LETTER LONG S folds to s
        return c;
    };
    // 1. contractions
    if (P(i) == '\'') {
        uint32_t a = low(P(i + 1)), b = low(P(i + 2));
        if (a == 's' || a == 't') return 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e')) return 3;
        if (a == 'm') return 2;
        if (a == 'l' && b == 'l') return 3;
        if (a == 'd') return 2;
    }
    auto is_crlf = [&](size_t j) { return P(j) == '\r' || P(j) == '\n'; };
    if (fam == kSplitGPT2) {
        for (int want : {0, 1, 3}) {            //  ?\p{L}+ |  ?\p{N}+ |  ?[^\s\p{L}\p{N}]+
            size_t j = i;
            if (P(j) == ' ' && C(j + 1) == want) ++j;
            if (C(j) == want) { while (C(j) == want) ++j; return j - i; }
        }
    } else {
        // 2. [^\r\n\p{L}\p{N}]?\p{L}+
        {
            size_t j = i;
            int c0 = C(j);
            if ((c0 == 2 || c0 == 3) && !is_crlf(j) && C(j + 1) == 0) ++j;
            if (C(j) == 0) { while (C(j) == 0) ++j; return j - i; }
        }
        // 3. \p{N}{1,3}  /  \p{N}
        if (C(i) == 1) {
            size_t cap = fam == kSplitLlama3 ? 3 : 1, j = i;
            while (j - i < cap && C(j) == 1) ++j;
            return j - i;
        }
        // 4.  ?[^\s\p{L}\p{N}]+[\r\n]*
        {
            size_t j = i;
            if (P(j) == ' ' && C(j + 1) == 3) ++j;
            if (C(j) == 3) {
                while (C(j) == 3) ++j;
                while (is_crlf(j)) ++j;
                return j - i;
            }
        }
        // 5. \s*[\r\n]+
        if (C(i) == 2) {
            size_t e = i;
            while (C(e) == 2) ++e;
            size_t last = e;
            while (last > i && !is_crlf(last - 1)) --last;
            if (last > i) return last - i;
        }
    }
    // \s+(?!\S) | \s+
    size_t e = i;
    while (C(e) == 2) ++e;
    if (e > i) {
        if (e == n) return e - i;
        if (e - i >= 2) return e - i - 1;
        return 1;
    }
    return 1;   // unreachable for valid input: every codepoint is in one of the classes
}

// ---- DeepSeek-V3 ----
// Wide class of a codepoint: 0 \p{L} or \p{M}, 1 \p{N}, 2 \s, 3 other, 6 \p{P} or \p{S}.
inline int wide_class(uint32_t cp) { return static_cast<int>(gtok_uw_lookup(gtok_uw_stage1_init, gtok_uw_stage2_init, cp)); }
inline bool ds_cjk(uint32_t cp) { return (cp >= 0x4E00 && cp <= 0x9FA5) || (cp >= 0x3040 && cp <= 0x309F) || (cp >= 0x30A0 && cp <= 0x30FF); }

// Length of the main pattern's match at cursor i of the piece [i, end), 0 when no alternative matches.
inline size_t ds_main_match(const std::vector<uint32_t>& cp, const std::vector<int>& wc, size_t i, size_t end) {
    auto K = [&](size_t j) -> int { return j < end ? wc[j] : -1; };
    auto P = [&](size_t j) -> uint32_t { return j < end ? cp[j] : 0xFFFFFFFFu; };
    auto letter = [&](size_t j) { uint32_t c = P(j); return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z'); };
    auto nl = [&](size_t j) { return P(j) == '\r' || P(j) == '\n'; };
    // punctuation of the ASCII range, then ASCII letters
    {
        uint32_t c = P(i);
        const bool punct = (c >= '!' && c <= '/') || (c >= ':' && c <= '@') || (c >= '[' && c <= '`') || (c >= '{' && c <= '~');
        if (punct && letter(i + 1)) { size_t j = i + 1; while (letter(j)) ++j; return j - i; }
    }
    // one optional codepoint that is no newline, letter, punctuation or symbol; then letters and marks
    {
        size_t j = i;
        if (K(j) != 0 && K(j) != 6 && !nl(j) && K(j + 1) == 0) ++j;
        if (K(j) == 0) { while (K(j) == 0) ++j; return j - i; }
    }
    // an optional space, punctuation and symbols, then newlines
    {
        size_t j = i;
        if (P(j) == ' ' && K(j + 1) == 6) ++j;
        if (K(j) == 6) { while (K(j) == 6) ++j; while (nl(j)) ++j; return j - i; }
    }
    size_t e = i;
    while (K(e) == 2) ++e;
    if (e == i) return 0;
    size_t last = e;
    while (last > i && !nl(last - 1)) --last;
    if (last > i) return last - i;               // \s*[\r\n]+
    if (e == end) return e - i;                  // \s+(?!\S) at the piece's end
    if (e - i >= 2) return e - i - 1;            // \s+(?!\S) before a non-space
    return 1;                                    // \s+
}

inline void split_deepseek(const Decoded& d, std::vector<uint32_t>& starts) {
    const size_t n = d.cp.size();
    std::vector<int> wc(n);
    for (size_t i = 0; i < n; ++i) wc[i] = wide_class(d.cp[i]);
    // the third step over one piece
    auto step3 = [&](size_t x, size_t y) {
        size_t i = x;
        bool gap = false;
        while (i < y) {
            const size_t m = ds_main_match(d.cp, wc, i, y);
            if (m) { starts.push_back(d.at[i]); i += m; gap = false; }
            else { if (!gap) starts.push_back(d.at[i]); gap = true; ++i; }
        }
    };
    // the second step over one piece
    auto step2 = [&](size_t a, size_t b) {
        size_t x = a;
        while (x < b) {
            size_t y = x;
            if (ds_cjk(d.cp[x])) { while (y < b && ds_cjk(d.cp[y])) ++y; }
            else { while (y < b && !ds_cjk(d.cp[y])) ++y; }
            step3(x, y);
            x = y;
        }
    };
    size_t a = 0;
    while (a < n) {
        if (wc[a] == 1) {
            size_t b = a;
            while (b < n && b - a < 3 && wc[b] == 1) ++b;
            starts.push_back(d.at[a]);           // a number piece; the later patterns match nothing in it
            a = b;
        } else {
            size_t b = a;
            while (b < n && wc[b] != 1) ++b;
            step2(a, b);
            a = b;
        }
    }
}

// Byte offsets at which pre-tokens start (no added-token handling).
inline void split(const uint8_t* s, size_t n, SplitFamily fam, std::vector<uint32_t>& starts) {
    Decoded d;
    decode_utf8(s, n, d);
    starts.clear();
    if (fam == kSplitDeepSeek) { split_deepseek(d, starts); return; }
    size_t i = 0;
    while (i < d.cp.size()) {
        starts.push_back(d.at[i]);
        i += match_at(d, i, fam);
    }
}

}  // namespace gtok_datagen
