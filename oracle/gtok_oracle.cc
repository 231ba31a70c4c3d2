// TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's encode path,
// used as the checker by tests/, by the smoke run and by the CPU-baseline leg
// of the benchmark.  Nothing in the shipped library calls into this file.
//
// It follows the reference's host encoder stage by stage
// (src/host_encode.cc:709-908 HostEncoder::encode):
//   1. dense per-codepoint arrays: class, first byte, byte position, and one
//      entry per added-token literal                      (host_encode.cc:725-800)
//   2. digit-run starts for the Llama-3 \p{N}{1,3} rule    (host_encode.cc:802-820)
//   3. a boundary predicate evaluated per codepoint        (src/pretok_boundary.h)
//   4. greedy lowest-rank-first BPE per pre-token          (host_encode.cc:558-648)
// The predicates are written from the regular expressions' semantics with the
// same decomposition into helper questions the reference uses
// (pretok_boundary.h:224-297 GPT-2, :515-671 Llama-3 / Qwen2.5); the local
// fast paths of the reference are an optimisation and are not restated.
//
// DeepSeek-V3 (three Split steps one after the other, src/vocab.cc:132-137 of the reference) has
// no host encoder in the reference (src/host_encode.cc:951-953 builds one for the other three
// families only); its restatement here reads the three patterns literally, as a scanner that
// tries the alternatives in order at each position, and is pinned against Hugging Face
// `tokenizers` alone.
//
// Parity pinning: tests/test_oracle_pin.py checks this file against (a) the
// reference's own HostEncoder compiled from its sources (oracle/_ref, when
// present), and (b) golden vectors produced by Hugging Face `tokenizers`
// (tests/golden/).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

#include "../graphtok_b200/csrc/unicode_class_table.h"
#include "../graphtok_b200/csrc/unicode_wide_table.h"
#include "../graphtok_b200/csrc/vocab_host.h"

namespace {

enum : uint8_t { kL = 0, kN = 1, kS = 2, kO = 3, kAdded = 5, kP = 6 };   // kP: \p{P} or \p{S}, wide table only
constexpr uint32_t kNone = 0xFFFFFFFFu;

// Lenient UTF-8 decode, exactly the reference's rule (pretok_boundary.h:43-57):
// the lead byte alone decides the width when enough bytes remain; continuation
// bytes are not validated; anything else is a one-byte codepoint.
uint32_t decode_lenient(const uint8_t* p, size_t avail) {
    uint8_t b = p[0];
    if (b < 0x80) return b;
    if ((b & 0xE0) == 0xC0 && avail >= 2) return ((b & 0x1Fu) << 6) | (p[1] & 0x3Fu);
    if ((b & 0xF0) == 0xE0 && avail >= 3) return ((b & 0x0Fu) << 12) | ((p[1] & 0x3Fu) << 6) | (p[2] & 0x3Fu);
    if ((b & 0xF8) == 0xF0 && avail >= 4)
        return ((b & 0x07u) << 18) | ((p[1] & 0x3Fu) << 12) | ((p[2] & 0x3Fu) << 6) | (p[3] & 0x3Fu);
    return b;
}

struct PairHash {
    size_t operator()(uint64_t k) const {
        k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33;
        return static_cast<size_t>(k);
    }
};

struct Oracle {
    gtok::HostVocab hv;
    // (left << 32 | right) -> (rank << 32 | result); first rule wins on a
    // repeated pair, as in the reference's insert-then-linear-probe table
    // (vocab.cc:745-795).
    std::unordered_map<uint64_t, uint64_t, PairHash> rules;
    std::unordered_map<std::string, uint32_t> whole;      // ignore_merges lookup
    std::unordered_map<std::string, uint32_t> literals;   // added tokens
    bool root_byte[256] = {};

    // ---- per-call dense arrays (stage 1) ----
    std::vector<uint8_t> cls, b0;
    std::vector<uint32_t> pos, direct, drun;
    uint32_t n = 0;

    // Accessors clamp to [0, n) and make an added-token entry look like the edge
    // of the text, as cls_at / b0_at do (pretok_boundary.h:76-85).
    int C(int j) const { return (j < 0 || static_cast<uint32_t>(j) >= n || cls[j] == kAdded) ? -1 : cls[j]; }
    int B(int j) const { return (j < 0 || static_cast<uint32_t>(j) >= n) ? -1 : b0[j]; }
    bool crlf(int j) const { int b = B(j); return b == 0x0D || b == 0x0A; }

    template <bool CI>
    int tail_len(int j) const {   // pretok_boundary.h:94-103
        int a = B(j), b = B(j + 1);
        if (CI) { if (a >= 'A' && a <= 'Z') a += 32; if (b >= 'A' && b <= 'Z') b += 32; }
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 2;
        if (a == 's' || a == 't' || a == 'm' || a == 'd') return 1;
        return 0;
    }

    // ------------------------------------------------------------------ GPT-2
    bool g_ws_split_before_last(int k) const {   // pretok_boundary.h:237-240
        return C(k) == kS && C(k + 1) >= 0 && C(k + 1) != kS && C(k - 1) == kS;
    }
    bool g_ws_last_attaches(int k) const {       // :241-244
        return C(k) == kS && C(k + 1) >= 0 && C(k + 1) != kS && B(k) == 0x20;
    }
    int g_starts(int k) const {                  // :250-261
        if (B(k) != 0x27) return 0;
        int tl = tail_len<false>(k + 1);
        if (!tl) return 0;
        if (k == 0) return tl;
        int p = C(k - 1);
        if (p == kO) return 0;
        if (p == kS && B(k - 1) == 0x20 && g_ws_last_attaches(k - 1)) return 0;
        return tl;
    }
    bool g_in_tail(int k) const { return g_starts(k - 1) >= 1 || g_starts(k - 2) == 2; }
    bool gpt2_boundary(int c) const {            // :224-297
        if (cls[c] == kAdded || c == 0) return true;
        int prev = C(c - 1), cur = C(c);
        bool cont;
        if (g_in_tail(c)) cont = true;
        else if (g_starts(c)) cont = false;
        else if (g_ws_last_attaches(c - 1) && (cur == kL || cur == kN || cur == kO)) cont = true;
        else if (cur == kS) cont = g_ws_split_before_last(c) ? false : prev == kS;
        else if (cur == prev && (cur == kL || cur == kN || cur == kO)) {
            // A letter directly after a finished contraction starts afresh.
            bool after_tail = g_starts(c - 2) == 1 || g_starts(c - 3) == 2;
            cont = !g_in_tail(c - 1) && !(cur == kL && after_tail);
        } else cont = false;
        return !cont;
    }

    // --------------------------------------------------------- Llama-3 / Qwen
    bool crlf_in_orun(int k) const {             // :533-539
        if (!crlf(k)) return false;
        int j = k - 1;
        while (j >= 0 && crlf(j)) --j;
        return j >= 0 && C(j) == kO;
    }
    bool in_ws_run(int k) const { return C(k) == kS && !crlf_in_orun(k); }
    bool o_attaches_letter(int k) const {        // :545-553
        if (C(k) != kO || C(k + 1) != kL) return false;
        if (k == 0) return true;
        int pc = C(k - 1);
        if (pc == kO) return false;
        if (pc == kS && B(k - 1) == 0x20) return false;
        return true;
    }
    void ws_run(int k, int& a, int& b, int& nl) const {
        a = k; while (a - 1 >= 0 && in_ws_run(a - 1)) --a;
        b = k; while (static_cast<uint32_t>(b) < n && in_ws_run(b)) ++b;
        nl = -1;
        for (int j = b - 1; j >= a; --j) if (crlf(j)) { nl = j; break; }
    }
    bool ws_continue(int k) const {              // :557-581
        int a, b, nl; ws_run(k, a, b, nl);
        int r = nl >= 0 ? nl + 1 : a;
        if (nl >= 0 && k > a && k <= nl) return true;
        if (k < r) return false;
        if (r >= b) return false;
        if (k == r) return false;
        if (C(b) < 0) return k > r;
        int last = b - 1;
        if (k == last) return false;
        return k > r && k < last;
    }
    bool ws_last_attaches(int k) const {         // :583-597
        int a, b, nl; ws_run(k, a, b, nl);
        if (C(b) < 0) return false;
        int r = nl >= 0 ? nl + 1 : a, last = b - 1;
        if (k != last || last < r) return false;
        int nxt = C(b), ch = B(last);
        if (nxt == kL && !crlf(last)) return true;
        if (nxt == kO && ch == 0x20) return true;
        return false;
    }
    int l_starts(int k) const {                  // :601-612
        if (B(k) != 0x27) return 0;
        int tl = tail_len<true>(k + 1);
        if (!tl) return 0;
        if (k == 0) return tl;
        int p = C(k - 1);
        if (p == kO) return 0;
        if (p == kS && B(k - 1) == 0x20 && ws_last_attaches(k - 1)) return 0;
        return tl;
    }
    bool l_in_tail(int k) const { return l_starts(k - 1) >= 1 || l_starts(k - 2) == 2; }
    template <bool DigitCap>
    bool llamaqwen_boundary(int c) const {       // :515-671
        if (cls[c] == kAdded || c == 0) return true;
        int prev = C(c - 1), cur = C(c);
        // Interior of a homogeneous whitespace stretch: decided without
        // rebuilding the run, so a very long run stays linear (:631-639).
        if (cur == kS && prev == kS) {
            if (crlf(c) && crlf(c - 1)) return false;
            if (!crlf(c) && !crlf(c - 1) && C(c + 1) == kS && !crlf(c + 1)) return false;
        }
        bool cont = false;
        if (l_in_tail(c)) cont = true;
        else if (l_starts(c)) cont = false;
        else if (crlf_in_orun(c)) cont = true;
        else if (cur == kS) cont = ws_continue(c);
        else if (cur == kL) {
            if (prev == kL && !l_in_tail(c - 1)) {
                bool after_tail = l_starts(c - 2) == 1 || l_starts(c - 3) == 2;
                cont = !after_tail;
            } else if (prev == kS && ws_last_attaches(c - 1)) cont = true;
            else if (prev == kO && o_attaches_letter(c - 1)) cont = true;
        } else if (cur == kN) {
            if (DigitCap) cont = prev == kN && ((c - drun[c]) % 3u) != 0u;
        } else if (cur == kO) {
            if (prev == kO && !o_attaches_letter(c)) cont = true;
            else if (prev == kS && B(c - 1) == 0x20 && ws_last_attaches(c - 1)) cont = true;
        }
        return !cont;
    }

    // ------------------------------------------------------------ DeepSeek-V3
    // Split(\p{N}{1,3}), then Split([一-龥぀-ゟ゠-ヿ]+), then Split(main pattern), each "Isolated":
    // every match is a piece and so is every stretch between two matches; a later step works on
    // each piece by itself, so a piece's two ends are the start and the end of the text for it.
    // cls holds the wide classes here (kL = \p{L} or \p{M}, kP = \p{P} or \p{S}); cpv the codepoints.
    std::vector<uint32_t> cpv;
    static bool is_cjk(uint32_t cp) { return (cp >= 0x4E00u && cp <= 0x9FA5u) || (cp >= 0x3040u && cp <= 0x30FFu); }
    static bool is_ascii_letter(uint32_t cp) { return (cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z'); }
    static bool is_ascii_punct(uint32_t cp) {
        return (cp >= 0x21 && cp <= 0x2F) || (cp >= 0x3A && cp <= 0x40) || (cp >= 0x5B && cp <= 0x60) || (cp >= 0x7B && cp <= 0x7E);
    }
    // The main pattern over codepoints [x, y): marks the start of every match and of every
    // stretch no alternative matches.
    void deepseek_main(uint32_t x, uint32_t y, std::vector<uint8_t>& bnd) const {
        auto nl = [&](uint32_t j) { return cpv[j] == 0x0D || cpv[j] == 0x0A; };
        uint32_t i = x;
        bool in_gap = false;
        while (i < y) {
            uint32_t end = 0;      // end of the match starting at i, 0 = none
            const uint8_t c = cls[i];
            // [!-/:-@\[-`{-~][A-Za-z]+
            if (is_ascii_punct(cpv[i]) && i + 1 < y && is_ascii_letter(cpv[i + 1])) {
                end = i + 2;
                while (end < y && is_ascii_letter(cpv[end])) ++end;
            }
            // [^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+
            if (!end) {
                uint32_t k = i;
                if (c != kL && c != kP && !nl(i) && i + 1 < y && cls[i + 1] == kL) k = i + 1;
                if (cls[k] == kL) { end = k + 1; while (end < y && cls[end] == kL) ++end; }
            }
            //  ?[\p{P}\p{S}]+[\r\n]*
            if (!end) {
                uint32_t k = i;
                if (cpv[i] == 0x20 && i + 1 < y && cls[i + 1] == kP) k = i + 1;
                if (cls[k] == kP) {
                    end = k + 1;
                    while (end < y && cls[end] == kP) ++end;
                    while (end < y && nl(end)) ++end;
                }
            }
            if (!end && c == kS) {
                uint32_t j = i;
                while (j < y && cls[j] == kS) ++j;
                // \s*[\r\n]+ : through the last newline of the run
                for (uint32_t l = j; l > i; --l) if (nl(l - 1)) { end = l; break; }
                // \s+(?!\S) : the whole run at the end of the piece, else all but its last codepoint
                if (!end) { if (j == y) end = j; else if (j - i >= 2) end = j - 1; }
                // \s+
                if (!end) end = j;
            }
            if (end) { bnd[i] = 1; i = end; in_gap = false; }
            else { if (!in_gap) bnd[i] = 1; in_gap = true; ++i; }
        }
    }
    void deepseek_bounds(std::vector<uint8_t>& bnd) const {
        bnd.assign(n, 0);
        uint32_t s = 0;
        while (s < n) {
            if (cls[s] == kAdded) { bnd[s] = 1; ++s; continue; }
            uint32_t e = s;
            while (e < n && cls[e] != kAdded) ++e;
            // step 1 over [s, e): runs of \p{N} in threes, the stretches between them go on
            uint32_t a = s;
            while (a < e) {
                if (cls[a] == kN) {
                    uint32_t b = a;
                    while (b < e && cls[b] == kN) ++b;
                    for (uint32_t j = a; j < b; j += 3) bnd[j] = 1;
                    a = b;
                    continue;
                }
                uint32_t b = a;
                while (b < e && cls[b] != kN) ++b;
                // step 2 over [a, b): runs inside and outside the three ranges
                uint32_t x = a;
                while (x < b) {
                    const bool cj = is_cjk(cpv[x]);
                    uint32_t y = x;
                    while (y < b && is_cjk(cpv[y]) == cj) ++y;
                    deepseek_main(x, y, bnd);     // step 3 (x itself is marked: a match or a gap starts there)
                    x = y;
                }
                a = b;
            }
            s = e;
        }
    }

    // ------------------------------------------------------------------- BPE
    bool rule(uint32_t l, uint32_t r, uint32_t& rank, uint32_t& res) const {
        auto it = rules.find((static_cast<uint64_t>(l) << 32) | r);
        if (it == rules.end()) return false;
        rank = static_cast<uint32_t>(it->second >> 32);
        res = static_cast<uint32_t>(it->second);
        return true;
    }

    // Greedy BPE: repeatedly merge the adjacent pair of lowest rank, leftmost
    // among equals, until no adjacent pair has a rule (host_encode.cc:617-648;
    // the heap form follows :558-607 and gives the same sequence).
    void bpe(const uint8_t* bytes, uint32_t len, std::vector<uint32_t>& out) const {
        if (hv.ignore_merges) {
            auto it = whole.find(std::string(reinterpret_cast<const char*>(bytes), len));
            if (it != whole.end()) { out.push_back(it->second); return; }
        }
        if (len < 64) {
            uint32_t sym[64], rk[64], nw[64];
            uint32_t m = len;
            for (uint32_t i = 0; i < m; ++i) sym[i] = hv.byte_to_id[bytes[i]];
            for (uint32_t i = 0; i + 1 < m; ++i) if (!rule(sym[i], sym[i + 1], rk[i], nw[i])) rk[i] = kNone;
            for (;;) {
                uint32_t best = kNone, bi = 0;
                for (uint32_t i = 0; i + 1 < m; ++i) if (rk[i] < best) { best = rk[i]; bi = i; }
                if (best == kNone) break;
                sym[bi] = nw[bi];
                for (uint32_t i = bi + 1; i + 1 < m; ++i) { sym[i] = sym[i + 1]; rk[i] = rk[i + 1]; nw[i] = nw[i + 1]; }
                --m;
                if (bi + 1 < m) { if (!rule(sym[bi], sym[bi + 1], rk[bi], nw[bi])) rk[bi] = kNone; }
                if (bi > 0) { if (!rule(sym[bi - 1], sym[bi], rk[bi - 1], nw[bi - 1])) rk[bi - 1] = kNone; }
            }
            out.insert(out.end(), sym, sym + m);
            return;
        }
        struct Cand { uint32_t rank, at, res, gen; };
        auto later = [](const Cand& x, const Cand& y) { return x.rank != y.rank ? x.rank > y.rank : x.at > y.at; };
        std::priority_queue<Cand, std::vector<Cand>, decltype(later)> heap(later);
        std::vector<uint32_t> sym(len), prv(len), nxt(len), gen(len, 0);
        for (uint32_t i = 0; i < len; ++i) {
            sym[i] = hv.byte_to_id[bytes[i]];
            prv[i] = i ? i - 1 : kNone;
            nxt[i] = i + 1 < len ? i + 1 : kNone;
        }
        auto offer = [&](uint32_t i) {
            if (nxt[i] == kNone) return;
            uint32_t rk, res;
            if (rule(sym[i], sym[nxt[i]], rk, res)) heap.push({rk, i, res, gen[i]});
        };
        for (uint32_t i = 0; i + 1 < len; ++i) offer(i);
        while (!heap.empty()) {
            Cand c = heap.top(); heap.pop();
            uint32_t i = c.at;
            if (gen[i] != c.gen || nxt[i] == kNone) continue;
            uint32_t j = nxt[i], k = nxt[j];
            sym[i] = c.res;
            nxt[i] = k;
            if (k != kNone) prv[k] = i;
            gen[j] = kNone;
            ++gen[i];
            uint32_t pv = prv[i];
            if (pv != kNone) ++gen[pv];
            offer(i);
            if (pv != kNone) offer(pv);
        }
        for (uint32_t i = 0; i != kNone; i = nxt[i]) out.push_back(sym[i]);
    }

    // Longest added-token literal starting at text[i], or 0.
    uint32_t match_literal(const uint8_t* text, size_t len, size_t i, uint32_t* id) const {
        uint32_t best = 0;
        size_t maxl = std::min<size_t>(hv.added_max_bytes, len - i);
        std::string key;
        for (size_t l = 1; l <= maxl; ++l) {
            key.assign(reinterpret_cast<const char*>(text + i), l);
            auto it = literals.find(key);
            if (it != literals.end()) { best = static_cast<uint32_t>(l); *id = it->second; }
        }
        return best;
    }

    // ---------------------------------------------------------------- Gemma-3 shape
    // What Hugging Face does with such a file: every space becomes U+2581, the Split on " " then finds nothing to
    // split, and the BPE model merges the characters of the whole text (between added tokens), lowest rank first,
    // leftmost among equals; a character the vocabulary lacks is spelt as its "<0xNN>" byte tokens, which no rule
    // mentions.  Done here on the characters themselves, with the file's own rules only (the loader's byte-level
    // rewriting is the product's business), one priority queue over the whole stretch.
    std::unordered_map<uint64_t, uint64_t, PairHash> sp_rules;      // the file's rules only, ranks from 0
    static size_t sp_char(const uint8_t* p, size_t avail, uint32_t* cp) {   // strict UTF-8, 0 = not a character
        const uint8_t c = p[0];
        if (c < 0x80) { *cp = c; return 1; }
        auto cont = [&](size_t k) { return k < avail && (p[k] & 0xC0) == 0x80; };
        if (c >= 0xC2 && c <= 0xDF && cont(1)) { *cp = ((c & 0x1Fu) << 6) | (p[1] & 0x3Fu); return 2; }
        if ((c & 0xF0) == 0xE0 && cont(1) && cont(2)) {
            *cp = ((c & 0x0Fu) << 12) | ((p[1] & 0x3Fu) << 6) | (p[2] & 0x3Fu);
            return (*cp >= 0x800 && !(*cp >= 0xD800 && *cp <= 0xDFFF)) ? 3 : 0;
        }
        if (c >= 0xF0 && c <= 0xF4 && cont(1) && cont(2) && cont(3)) {
            *cp = ((c & 0x07u) << 18) | ((p[1] & 0x3Fu) << 12) | ((p[2] & 0x3Fu) << 6) | (p[3] & 0x3Fu);
            return (*cp >= 0x10000 && *cp <= 0x10FFFF) ? 4 : 0;
        }
        return 0;
    }
    bool sp_id_of(uint32_t cp, uint32_t* id) const {
        auto it = std::lower_bound(hv.sp_chars.begin(), hv.sp_chars.end(), std::make_pair(cp, 0u));
        if (it == hv.sp_chars.end() || it->first != cp) return false;
        *id = it->second;
        return true;
    }
    void sp_segment(const uint8_t* text, size_t len, size_t base, std::vector<uint32_t>& out, std::vector<uint32_t>* starts) {
        std::vector<uint32_t> sym, cps;
        std::vector<uint32_t> at;                       // byte offset of each symbol
        std::vector<uint8_t> known;
        for (size_t i = 0; i < len;) {
            uint32_t cp = 0, id = 0;
            const size_t w = sp_char(text + i, len - i, &cp);
            if (w && sp_id_of(cp, &id)) { sym.push_back(id); cps.push_back(cp); known.push_back(1); at.push_back(static_cast<uint32_t>(base + i)); i += w; }
            else { sym.push_back(hv.sp_fallback[text[i]]); cps.push_back(0); known.push_back(0); at.push_back(static_cast<uint32_t>(base + i)); i += 1; }
        }
        const size_t m = sym.size();
        if (starts) {
            // where the product may cut (and does): around every byte that is not part of a character of the vocabulary,
            // and in front of a space unless a rule could join it to the character before
            for (size_t k = 0; k < m; ++k) {
                bool cut = k == 0 || !known[k] || !known[k - 1];
                if (!cut && (cps[k] == 0x20 || cps[k] == 0x2581)) cut = !std::binary_search(hv.sp_before_bar.begin(), hv.sp_before_bar.end(), cps[k - 1]);
                if (cut) starts->push_back(at[k]);
            }
        }
        std::vector<int> prev(m), next(m);
        std::vector<uint8_t> dead(m, 0);
        for (size_t k = 0; k < m; ++k) { prev[k] = static_cast<int>(k) - 1; next[k] = k + 1 < m ? static_cast<int>(k + 1) : -1; }
        struct Cand { uint32_t rank; uint32_t pos; uint32_t l, r, res; };
        auto worse = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.pos > b.pos; };
        std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
        auto push = [&](int k) {
            if (k < 0 || next[k] < 0) return;
            auto it = sp_rules.find((static_cast<uint64_t>(sym[k]) << 32) | sym[next[k]]);
            if (it != sp_rules.end()) heap.push({static_cast<uint32_t>(it->second >> 32), static_cast<uint32_t>(k), sym[k], sym[next[k]], static_cast<uint32_t>(it->second)});
        };
        for (size_t k = 0; k < m; ++k) push(static_cast<int>(k));
        while (!heap.empty()) {
            const Cand c = heap.top();
            heap.pop();
            const int k = static_cast<int>(c.pos);
            if (dead[k] || next[k] < 0 || sym[k] != c.l || sym[next[k]] != c.r) continue;     // stale
            const int r = next[k];
            sym[k] = c.res;
            dead[r] = 1;
            next[k] = next[r];
            if (next[r] >= 0) prev[next[r]] = k;
            push(prev[k]);
            push(k);
        }
        for (int k = m ? 0 : -1; k >= 0; k = next[k]) out.push_back(sym[k]);
    }
    void encode_sp(const uint8_t* text, size_t len, std::vector<uint32_t>& out, std::vector<uint32_t>* starts) {
        size_t seg = 0;
        for (size_t i = 0; i < len;) {
            uint32_t id = 0;
            const uint32_t al = (hv.added_max_bytes && root_byte[text[i]]) ? match_literal(text, len, i, &id) : 0u;
            if (!al) { ++i; continue; }
            if (i > seg) sp_segment(text + seg, i - seg, seg, out, starts);
            if (starts) starts->push_back(static_cast<uint32_t>(i));
            out.push_back(id);
            i += al;
            seg = i;
        }
        if (len > seg) sp_segment(text + seg, len - seg, seg, out, starts);
    }

    // Stage 1-3 of the encoder.  Fills `starts` with the byte offset of every
    // pre-token (added-token literals included) when `starts` is non-null.
    void encode(const uint8_t* text, size_t len, std::vector<uint32_t>& out, std::vector<uint32_t>* starts) {
        if (len == 0) return;
        if (hv.family == gtok::Family::Gemma3) { encode_sp(text, len, out, starts); return; }
        cls.resize(len); b0.resize(len); pos.resize(len); direct.resize(len);
        n = 0;
        const bool deepseek = hv.family == gtok::Family::DeepSeekV3;
        if (deepseek) cpv.resize(len);
        const bool fold = hv.family == gtok::Family::Llama3 || hv.family == gtok::Family::Qwen25;   // U+017F counts as 's' under (?i:)
        size_t i = 0;
        while (i < len) {
            uint8_t b = text[i];
            if (hv.added_max_bytes && root_byte[b]) {
                uint32_t id = 0, al = match_literal(text, len, i, &id);
                if (al) { cls[n] = kAdded; b0[n] = 0; pos[n] = static_cast<uint32_t>(i); direct[n] = id; ++n; i += al; continue; }
            }
            if ((b & 0xC0u) == 0x80u) { ++i; continue; }   // starts no codepoint
            uint32_t cp = decode_lenient(text + i, len - i);
            if (deepseek) {
                cls[n] = static_cast<uint8_t>(gtok_uw_lookup(gtok_uw_stage1_init, gtok_uw_stage2_init, cp));
                cpv[n] = cp;
            } else cls[n] = static_cast<uint8_t>(gtok_uc_lookup(gtok_uc_stage1_init, gtok_uc_stage2_init, cp));
            bool long_s = fold && b == 0xC5 && i + 1 < len && text[i + 1] == 0xBF;
            b0[n] = long_s ? static_cast<uint8_t>('s') : b;
            pos[n] = static_cast<uint32_t>(i);
            ++n; ++i;
        }
        if (n == 0) return;
        if (hv.family == gtok::Family::Llama3) {
            drun.resize(n);
            for (uint32_t c = 0; c < n;) {
                if (cls[c] != kN) { ++c; continue; }
                uint32_t s = c;
                do { drun[c] = s; ++c; } while (c < n && cls[c] == kN);
            }
        }
        std::vector<uint8_t> ds_bnd;
        if (deepseek) deepseek_bounds(ds_bnd);
        uint32_t start = 0;
        for (uint32_t c = 1; c <= n; ++c) {
            if (c < n) {
                bool bnd;
                switch (hv.family) {
                    case gtok::Family::DeepSeekV3: bnd = ds_bnd[c] != 0; break;
                    case gtok::Family::GPT2: bnd = gpt2_boundary(static_cast<int>(c)); break;
                    case gtok::Family::Llama3: bnd = llamaqwen_boundary<true>(static_cast<int>(c)); break;
                    default: bnd = llamaqwen_boundary<false>(static_cast<int>(c)); break;
                }
                if (!bnd) continue;
            }
            if (starts) starts->push_back(pos[start]);
            if (cls[start] == kAdded) {
                out.push_back(direct[start]);
            } else {
                uint32_t sb = pos[start], eb = c < n ? pos[c] : static_cast<uint32_t>(len);
                bpe(text + sb, eb - sb, out);
            }
            start = c;
        }
    }
};

}  // namespace

extern "C" {

void* gtok_oracle_create(const char* tokenizer_json, char* err, uint32_t err_cap) {
    Oracle* o = new Oracle();
    std::string e;
    if (!gtok::load_tokenizer_json(tokenizer_json, o->hv, e)) {
        if (err && err_cap) { std::strncpy(err, e.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
        delete o;
        return nullptr;
    }
    for (uint32_t k = 0; k < o->hv.merges.size(); ++k) {
        const gtok::MergeRule& m = o->hv.merges[k];
        o->rules.emplace((static_cast<uint64_t>(m.left) << 32) | m.right, (static_cast<uint64_t>(k) << 32) | m.result);
    }
    for (uint32_t k = o->hv.sp_synthetic; k < o->hv.merges.size() && o->hv.family == gtok::Family::Gemma3; ++k) {
        const gtok::MergeRule& m = o->hv.merges[k];
        o->sp_rules.emplace((static_cast<uint64_t>(m.left) << 32) | m.right, (static_cast<uint64_t>(k - o->hv.sp_synthetic) << 32) | m.result);
    }
    if (o->hv.ignore_merges)
        for (uint32_t id = 0; id < o->hv.token_bytes.size(); ++id)
            if (!o->hv.token_bytes[id].empty()) o->whole.emplace(o->hv.token_bytes[id], id);
    for (const gtok::AddedToken& a : o->hv.added) {
        o->literals.emplace(a.content, a.id);
        o->root_byte[static_cast<unsigned char>(a.content[0])] = true;
    }
    return o;
}

void gtok_oracle_destroy(void* h) { delete static_cast<Oracle*>(h); }

// 0 GPT-2, 1 Llama-3, 2 Qwen2.5, 3 DeepSeek-V3, 4 Gemma-3; bit 8 set when the vocabulary asks for NFC.
uint32_t gtok_oracle_family(void* h) {
    Oracle* o = static_cast<Oracle*>(h);
    return static_cast<uint32_t>(o->hv.family) | (o->hv.nfc ? 0x100u : 0u);
}

// Encodes already-normalised bytes.  Returns the token count (which may exceed
// `cap`; only the first `cap` ids are written).  When `starts` is non-null it
// receives the byte offset of each pre-token, `*n_starts` their number.
int64_t gtok_oracle_encode(void* h, const uint8_t* text, uint64_t len, uint32_t* out, uint64_t cap,
                           uint32_t* starts, uint64_t starts_cap, uint64_t* n_starts) {
    Oracle* o = static_cast<Oracle*>(h);
    std::vector<uint32_t> ids, st;
    ids.reserve(len / 3 + 16);
    o->encode(text, len, ids, (starts || n_starts) ? &st : nullptr);
    size_t w = std::min<size_t>(ids.size(), cap);
    if (out && w) std::memcpy(out, ids.data(), w * sizeof(uint32_t));
    if (n_starts) *n_starts = st.size();
    if (starts) {
        size_t ws = std::min<size_t>(st.size(), starts_cap);
        if (ws) std::memcpy(starts, st.data(), ws * sizeof(uint32_t));
    }
    return static_cast<int64_t>(ids.size());
}

}  // extern "C"
