// See tables_build.h.
#include "tables_build.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <unordered_map>

namespace gtok {

namespace {

uint32_t pow2_at_least(uint64_t x) {
    uint32_t p = 16;
    while (p < x) p <<= 1;
    return p;
}

struct RuleMap {
    std::unordered_map<uint64_t, uint64_t> m;
    bool find(uint32_t l, uint32_t r, uint32_t& rank, uint32_t& res) const {
        auto it = m.find((static_cast<uint64_t>(l) << 32) | r);
        if (it == m.end()) return false;
        rank = static_cast<uint32_t>(it->second >> 32);
        res = static_cast<uint32_t>(it->second);
        return true;
    }
};

// Plain greedy BPE of a short byte string; used once per vocabulary token at
// load time to decide which tokens may enter the whole-word table.
bool merges_to_self(const HostVocab& hv, const RuleMap& rules, const std::string& bytes, uint32_t id) {
    std::vector<uint32_t> sym;
    for (unsigned char c : bytes) sym.push_back(hv.byte_to_id[c]);
    for (;;) {
        uint32_t best = kNoRank, bi = 0, bres = 0;
        for (size_t i = 0; i + 1 < sym.size(); ++i) {
            uint32_t rk, res;
            if (rules.find(sym[i], sym[i + 1], rk, res) && rk < best) { best = rk; bi = static_cast<uint32_t>(i); bres = res; }
        }
        if (best == kNoRank) break;
        sym[bi] = bres;
        sym.erase(sym.begin() + bi + 1);
    }
    return sym.size() == 1 && sym[0] == id;
}

}  // namespace

bool build_host_tables(const HostVocab& hv, HostTables& out, std::string& err) {
    out.family = static_cast<uint32_t>(hv.family);
    out.ignore_merges = hv.ignore_merges ? 1u : 0u;
    out.monotone = hv.monotone ? 1u : 0u;
    out.byte_to_id.assign(hv.byte_to_id, hv.byte_to_id + 256);

    // ---- merge rules ----------------------------------------------------
    if (hv.merges.size() >= (1u << 26) - 2u) { err = "more merge rules than the kernels' rank keys can hold (2^26)"; return false; }
    RuleMap rules;
    rules.m.reserve(hv.merges.size() * 2);
    for (uint32_t k = 0; k < hv.merges.size(); ++k) {
        const MergeRule& m = hv.merges[k];
        // The first rule for a pair wins; a later duplicate is unreachable in
        // the reference's table too (src/vocab.cc:745-795).
        rules.m.emplace((static_cast<uint64_t>(m.left) << 32) | m.right, (static_cast<uint64_t>(k) << 32) | m.result);
    }
    // Buckets of two slots, at least four slots per rule.  A rule goes to its first bucket when that has
    // room, else to its second; when both are full one occupant of the first bucket moves over to its own
    // other bucket, and so on; a walk that does not end soon means a cycle, and the table is rebuilt at
    // twice the size.  Afterwards every bucket that is the FIRST bucket of a rule living elsewhere is flagged.
    for (uint32_t bits = 4;; ++bits) {
        if (bits > 30) { err = "merge table cannot be built"; return false; }
        if ((1ull << bits) < static_cast<uint64_t>(hv.merges.size()) * 4) continue;
        const uint32_t shift = 32 - (bits - 1);                     // bits - 1 = log2(buckets)
        out.merge.assign(size_t(1) << bits, MergeSlot{kEmptyKey, kEmptyKey, kNoRank, 0});
        out.merge_shift = shift;
        auto free_slot = [&](uint32_t b) -> int {
            if (out.merge[2 * b].left == kEmptyKey) return 0;
            if (out.merge[2 * b + 1].left == kEmptyKey) return 1;
            return -1;
        };
        auto holds = [&](uint32_t b, uint32_t l, uint32_t r) {
            return (out.merge[2 * b].left == l && out.merge[2 * b].right == r) || (out.merge[2 * b + 1].left == l && out.merge[2 * b + 1].right == r);
        };
        bool ok = true;
        uint32_t turn = 0;
        for (uint32_t k = 0; k < hv.merges.size() && ok; ++k) {
            const MergeRule& m = hv.merges[k];
            uint32_t b1, b2;
            merge_buckets(m.left, m.right, shift, &b1, &b2);
            if (holds(b1, m.left, m.right) || holds(b2, m.left, m.right)) continue;    // a later duplicate of a pair is unreachable: keep the first
            MergeSlot cur{m.left, m.right, k, m.result};
            uint32_t at = b1;
            ok = false;
            for (int kicks = 0; kicks < 512; ++kicks) {
                int f = free_slot(at);
                if (f < 0) {
                    uint32_t c1, c2;
                    merge_buckets(cur.left, cur.right, shift, &c1, &c2);
                    const uint32_t other = at == c1 ? c2 : c1;
                    f = free_slot(other);
                    if (f >= 0) at = other;
                }
                if (f >= 0) { out.merge[2 * at + f] = cur; ok = true; break; }
                // both buckets full: take a slot of `at`, its occupant moves on to its own other bucket
                const uint32_t victim = 2 * at + (turn++ & 1u);
                std::swap(cur, out.merge[victim]);
                uint32_t c1, c2;
                merge_buckets(cur.left, cur.right, shift, &c1, &c2);
                at = at == c1 ? c2 : c1;
            }
        }
        if (!ok) continue;
        for (size_t i = 0; i < out.merge.size(); ++i) {
            const MergeSlot& sl = out.merge[i];
            if (sl.left == kEmptyKey) continue;
            uint32_t b1, b2;
            merge_buckets(sl.left, sl.right, shift, &b1, &b2);
            if ((i >> 1) != b1) out.merge[2 * static_cast<size_t>(b1)].result |= kBucketSpills;
        }
        break;
    }

    // ---- Gemma-3 shape: the vocabulary's characters as a class table ------------
    out.sp_stage1.clear();
    out.sp_stage2.clear();
    for (int i = 0; i < 4; ++i) out.sp_ascii_known[i] = out.sp_ascii_before_bar[i] = 0;
    if (hv.family == Family::Gemma3) {
        for (const auto& c : hv.sp_chars) if (c.first < 128) out.sp_ascii_known[c.first >> 5] |= 1u << (c.first & 31);
        for (uint32_t c : hv.sp_before_bar) if (c < 128) out.sp_ascii_before_bar[c >> 5] |= 1u << (c & 31);
        std::map<std::vector<uint32_t>, uint16_t> leaves;      // sixteen words of 4-bit classes -> leaf number
        out.sp_stage1.assign(0x110000 / 128, 0);
        size_t ci = 0, bi = 0;
        for (uint32_t block = 0; block < 0x110000 / 128; ++block) {
            std::vector<uint32_t> leaf(16, 0x33333333u);
            const uint32_t lo = block * 128, hi = lo + 128;
            while (ci < hv.sp_chars.size() && hv.sp_chars[ci].first < lo) ++ci;
            while (bi < hv.sp_before_bar.size() && hv.sp_before_bar[bi] < lo) ++bi;
            for (size_t k = ci; k < hv.sp_chars.size() && hv.sp_chars[k].first < hi; ++k) {
                const uint32_t o = hv.sp_chars[k].first - lo;
                leaf[o >> 3] &= ~(15u << ((o & 7) * 4));
            }
            for (size_t k = bi; k < hv.sp_before_bar.size() && hv.sp_before_bar[k] < hi; ++k) {
                const uint32_t o = hv.sp_before_bar[k] - lo;
                if (((leaf[o >> 3] >> ((o & 7) * 4)) & 15u) == 0) leaf[o >> 3] |= 6u << ((o & 7) * 4);
            }
            auto it = leaves.find(leaf);
            if (it == leaves.end()) {
                if (leaves.size() >= 0xFFFF) { err = "too many distinct blocks of characters"; return false; }
                it = leaves.emplace(leaf, static_cast<uint16_t>(leaves.size())).first;
                out.sp_stage2.insert(out.sp_stage2.end(), leaf.begin(), leaf.end());
            }
            out.sp_stage1[block] = it->second;
        }
    }

    // ---- whole-word table -------------------------------------------------
    std::vector<std::pair<std::string, uint32_t>> entries;   // (bytes, id)
    {
        std::map<std::string, uint32_t> lowest;   // the lowest id wins for a repeated spelling
        for (uint32_t id = 0; id < hv.token_bytes.size() && id < hv.vocab_size; ++id) {     // (ids beyond: partly assembled characters of a Gemma-3 vocabulary)
            const std::string& b = hv.token_bytes[id];
            if (b.empty()) continue;
            if (!hv.ignore_merges) {
                if (b.size() > static_cast<size_t>(kWordKeyMax)) continue;
                if (!merges_to_self(hv, rules, b, id)) continue;
            }
            lowest.emplace(b, id);
        }
        entries.assign(lowest.begin(), lowest.end());
    }
    size_t n_short = 0;
    for (const auto& e : entries) if (e.first.size() <= static_cast<size_t>(kWordKeyMax)) ++n_short;
    // eight slots per entry: one key in eight is then away from its home slot, and each of those
    // costs its thread a further dependent load while the rest of the block waits
    for (uint32_t cap = pow2_at_least(n_short * 8);; cap <<= 1) {
        if (cap > (1u << 28)) { err = "word table cannot be built within its probe limit"; return false; }
        out.word.assign(cap, WordSlot{0, 0, kNoToken, {0, 0, 0}});
        const uint32_t mask = cap - 1;
        bool ok = true;
        for (const auto& e : entries) {
            if (e.first.size() > static_cast<size_t>(kWordKeyMax)) continue;
            uint64_t k0, k1;
            make_word_key(reinterpret_cast<const uint8_t*>(e.first.data()), static_cast<uint32_t>(e.first.size()), k0, k1);
            uint32_t h = word_hash(k0, k1) & mask;
            int steps = 0;
            for (;; h = (h + 1) & mask) {
                WordSlot& s = out.word[h];
                if (s.id == kNoToken) { s.k0 = k0; s.k1 = k1; s.id = e.second; break; }
                if (++steps >= kProbeLimit - 1) { ok = false; break; }
            }
            if (!ok) break;
        }
        if (ok) break;
    }

    // ---- long-token table (ignore_merges) ---------------------------------
    out.longtab.clear();
    out.long_blob.clear();
    out.long_max_len = 0;
    if (hv.ignore_merges) {
        size_t n_long = entries.size() - n_short;
        for (uint32_t cap = pow2_at_least(n_long * 2);; cap <<= 1) {
            if (cap > (1u << 28)) { err = "long-token table cannot be built within its probe limit"; return false; }
            out.longtab.assign(cap, LongSlot{0, kNoToken, 0, 0, 0});
            out.long_blob.clear();
            const uint32_t mask = cap - 1;
            bool ok = true;
            for (const auto& e : entries) {
                if (e.first.size() <= static_cast<size_t>(kWordKeyMax)) continue;
                uint64_t h = kLongHashSeed;
                for (unsigned char c : e.first) h = long_hash_step(h, c);
                h = long_hash_finish(h, static_cast<uint32_t>(e.first.size()));
                uint32_t at = static_cast<uint32_t>(h) & mask;
                int steps = 0;
                for (;; at = (at + 1) & mask) {
                    LongSlot& s = out.longtab[at];
                    if (s.id == kNoToken) {
                        s.hash = h; s.id = e.second; s.off = static_cast<uint32_t>(out.long_blob.size());
                        s.len = static_cast<uint32_t>(e.first.size());
                        out.long_blob.insert(out.long_blob.end(), e.first.begin(), e.first.end());
                        while (out.long_blob.size() % 4) out.long_blob.push_back(0);        // spellings start on 4-byte boundaries, zero padded
                        out.long_max_len = std::max(out.long_max_len, s.len);
                        break;
                    }
                    if (++steps >= kProbeLimit - 1) { ok = false; break; }
                }
                if (!ok) break;
            }
            if (ok) break;
        }
    }
    out.long_blob.resize(out.long_blob.size() + 4, 0);
    if (out.longtab.empty()) out.longtab.assign(16, LongSlot{0, kNoToken, 0, 0, 0});

    // ---- added-token trie ---------------------------------------------------
    out.added_max_bytes = hv.added_max_bytes;
    out.added_ws = 0;
    out.added_alpha_end = 0;
    for (const AddedToken& a : hv.added) {
        for (unsigned char c : a.content) if (c == 0x20 || (c >= 0x09 && c <= 0x0D)) out.added_ws = 1;
        const unsigned char last = a.content.empty() ? 0 : static_cast<unsigned char>(a.content.back());
        if ((last >= 'a' && last <= 'z') || (last >= 'A' && last <= 'Z')) out.added_alpha_end = 1;
    }
    for (int i = 0; i < 8; ++i) out.lit1_bits[i] = out.lit2_bits[i] = 0;
    out.lit_single = 0;
    for (const auto& a : hv.added) {
        if (a.content.empty()) continue;
        const unsigned char c0 = static_cast<unsigned char>(a.content[0]);
        out.lit1_bits[c0 >> 5] |= 1u << (c0 & 31);
        if (a.content.size() == 1) { out.lit_single = 1; continue; }
        const unsigned char c1 = static_cast<unsigned char>(a.content[1]);
        out.lit2_bits[c1 >> 5] |= 1u << (c1 & 31);
    }
    // the distinct first bytes, when there are at most four of them (the usual case: '<'), packed one per byte
    {
        out.lit_first_n = 0;
        out.lit_first = 0;
        for (int b = 0; b < 256; ++b)
            if ((out.lit1_bits[b >> 5] >> (b & 31)) & 1u) {
                if (out.lit_first_n < 4) out.lit_first |= static_cast<uint32_t>(b) << (8 * out.lit_first_n);
                ++out.lit_first_n;
            }
    }
    // the same literals as a hash table (see device_tables.h)
    {
        std::vector<uint32_t> lens;
        bool fits = true;
        for (const auto& a : hv.added) {
            if (a.content.empty()) continue;
            lens.push_back(static_cast<uint32_t>(a.content.size()));
            if (a.content.size() > static_cast<size_t>(kLitInline)) fits = false;
        }
        std::sort(lens.begin(), lens.end());
        lens.erase(std::unique(lens.begin(), lens.end()), lens.end());
        out.lit_n_lens = (fits && lens.size() <= static_cast<size_t>(kLitLens)) ? static_cast<uint32_t>(lens.size()) : 0u;
        for (int i = 0; i < kLitLens; ++i) out.lit_lens[i] = static_cast<uint32_t>(i) < out.lit_n_lens ? lens[i] : 0u;
        LitSlot empty;
        std::memset(&empty, 0, sizeof empty);
        empty.id = kNoToken;
        out.littab.assign(16, empty);
        if (out.lit_n_lens) {
            for (uint32_t cap = pow2_at_least(hv.added.size() * 4 + 16);; cap <<= 1) {
                if (cap > (1u << 22)) { out.lit_n_lens = 0; out.littab.assign(16, empty); break; }
                out.littab.assign(cap, empty);
                const uint32_t mask = cap - 1;
                bool ok = true;
                for (const auto& a : hv.added) {
                    if (a.content.empty()) continue;
                    uint32_t h = 0, pk = kLitHashK;
                    for (unsigned char c : a.content) { h += c * pk; pk *= kLitHashK; }
                    h = lit_hash_finish(h, static_cast<uint32_t>(a.content.size()));
                    uint32_t at = h & mask;
                    int steps = 0;
                    for (;; at = (at + 1) & mask) {
                        LitSlot& sl = out.littab[at];
                        if (sl.id == kNoToken) {
                            sl.hash = h; sl.id = a.id; sl.len = static_cast<uint32_t>(a.content.size());
                            std::memcpy(sl.bytes, a.content.data(), a.content.size());
                            break;
                        }
                        if (sl.hash == h && sl.len == a.content.size() && std::memcmp(sl.bytes, a.content.data(), a.content.size()) == 0) {
                            sl.id = a.id;                     // a repeated literal: the last id stands, as in the trie
                            break;
                        }
                        if (++steps >= 4) { ok = false; break; }
                    }
                    if (!ok) break;
                }
                if (ok) break;
            }
        }
    }
    if (hv.added_max_bytes > kMaxAddedBytes) {
        err = "an added-token literal is longer than the on-device matcher supports";
        return false;
    }
    struct Node { std::map<uint8_t, uint32_t> next; uint32_t terminal = kNoToken; };
    std::vector<Node> nodes(1);
    for (const AddedToken& a : hv.added) {
        uint32_t at = 0;
        for (unsigned char c : a.content) {
            auto it = nodes[at].next.find(c);
            if (it == nodes[at].next.end()) {
                uint32_t fresh = static_cast<uint32_t>(nodes.size());
                nodes[at].next.emplace(c, fresh);
                nodes.emplace_back();
                at = fresh;
            } else at = it->second;
        }
        nodes[at].terminal = a.id;
    }
    // Path compression: a node reached by an edge swallows the chain of single-child,
    // non-terminal nodes below it as its skip string.
    out.trie_root.assign(256, kNoToken);
    out.trie_first.clear(); out.trie_count.clear(); out.trie_terminal.clear(); out.trie_edges.clear();
    out.trie_skip.clear(); out.trie_blob.clear();
    struct Pending { uint32_t plain, packed; };
    std::vector<Pending> work;
    auto add_packed = [&](uint32_t plain) -> uint32_t {
        const uint32_t off = static_cast<uint32_t>(out.trie_blob.size());
        uint32_t len = 0;
        while (nodes[plain].terminal == kNoToken && nodes[plain].next.size() == 1) {
            out.trie_blob.push_back(nodes[plain].next.begin()->first);
            plain = nodes[plain].next.begin()->second;
            ++len;
        }
        const uint32_t id = static_cast<uint32_t>(out.trie_skip.size());
        out.trie_skip.push_back((off << 8) | len);          // len <= kMaxAddedBytes < 256
        out.trie_terminal.push_back(nodes[plain].terminal);
        out.trie_first.push_back(0);
        out.trie_count.push_back(0);
        work.push_back(Pending{plain, id});
        return id;
    };
    for (const auto& e : nodes[0].next) out.trie_root[e.first] = add_packed(e.second);
    for (size_t w = 0; w < work.size(); ++w) {
        const Pending pd = work[w];
        const Node& nd = nodes[pd.plain];
        std::vector<uint32_t> edges;
        for (const auto& e : nd.next) edges.push_back((add_packed(e.second) << 8) | e.first);
        out.trie_first[pd.packed] = static_cast<uint32_t>(out.trie_edges.size());
        out.trie_count[pd.packed] = static_cast<uint16_t>(edges.size());
        out.trie_edges.insert(out.trie_edges.end(), edges.begin(), edges.end());
    }
    if (out.trie_blob.empty()) out.trie_blob.push_back(0);
    if (out.trie_skip.empty()) { out.trie_skip.push_back(0); out.trie_terminal.push_back(kNoToken); out.trie_first.push_back(0); out.trie_count.push_back(0); }
    if (out.trie_edges.empty()) out.trie_edges.push_back(0);
    return true;
}

}  // namespace gtok
