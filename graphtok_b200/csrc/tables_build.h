// Host-side construction of the device vocabulary tables (device_tables.h)
// from a HostVocab.  Pure C++: the result is a set of host vectors that the
// engine uploads verbatim, so the construction is testable without a GPU.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "device_tables.h"
#include "vocab_host.h"

namespace gtok {

struct HostTables {
    std::vector<MergeSlot> merge;
    uint32_t merge_shift = 0;
    std::vector<WordSlot> word;
    std::vector<LongSlot> longtab;
    std::vector<uint8_t> long_blob;
    uint32_t long_max_len = 0;
    std::vector<uint32_t> byte_to_id;
    std::vector<uint32_t> trie_root, trie_first, trie_terminal, trie_edges, trie_skip;
    std::vector<uint8_t> trie_blob;
    std::vector<uint16_t> trie_count;
    uint32_t added_max_bytes = 0;
    uint32_t lit1_bits[8] = {}, lit2_bits[8] = {}, lit_single = 0;
    std::vector<LitSlot> littab;
    uint32_t lit_n_lens = 0, lit_lens[kLitLens] = {};
    // Gemma-3 shape: a class per codepoint in the layout of the wide class table (uc_class(..., wide)), made from the
    // vocabulary: 0 a character of the vocabulary, 6 one that a rule may join to a U+2581 after it, 3 any other codepoint
    std::vector<uint16_t> sp_stage1;
    std::vector<uint32_t> sp_stage2;
    uint32_t sp_ascii_known[4] = {}, sp_ascii_before_bar[4] = {};
    uint32_t family = 0, ignore_merges = 0, monotone = 1, added_ws = 0, added_alpha_end = 0, lit_first = 0, lit_first_n = 0;
};

// Returns false (with a reason) when a table cannot be built within its probe
// limit or an added-token literal is too long for the on-device matcher.
bool build_host_tables(const HostVocab& hv, HostTables& out, std::string& err);

// The scalar fields of the device view of the tables (the pointers are set by whoever owns the arrays).
inline void fill_table_scalars(const HostTables& ht, DeviceTables& tb) {
    tb.merge_shift = ht.merge_shift;
    tb.word_mask = static_cast<uint32_t>(ht.word.size() - 1);
    tb.long_mask = static_cast<uint32_t>(ht.longtab.size() - 1);
    tb.long_max_len = ht.long_max_len;
    tb.added_max_bytes = ht.added_max_bytes;
    for (int i = 0; i < 8; ++i) { tb.lit1_bits[i] = ht.lit1_bits[i]; tb.lit2_bits[i] = ht.lit2_bits[i]; }
    tb.lit_single = ht.lit_single;
    tb.lit_mask = static_cast<uint32_t>(ht.littab.size() - 1);
    tb.lit_n_lens = ht.lit_n_lens;
    for (int i = 0; i < kLitLens; ++i) tb.lit_lens[i] = ht.lit_lens[i];
    tb.family = ht.family;
    for (int i = 0; i < 4; ++i) { tb.sp_ascii_known[i] = ht.sp_ascii_known[i]; tb.sp_ascii_before_bar[i] = ht.sp_ascii_before_bar[i]; }
    tb.uc_wide = ht.family == 3 || ht.family == 4 ? 1u : 0u;
    tb.ignore_merges = ht.ignore_merges;
    tb.monotone = ht.monotone;
    tb.added_ws = ht.added_ws;
    tb.added_alpha_end = ht.added_alpha_end;
    tb.lit_first = ht.lit_first;
    tb.lit_first_n = ht.lit_first_n;
}

// Packs up to 15 bytes into a word-table key.
inline void make_word_key(const uint8_t* bytes, uint32_t len, uint64_t& k0, uint64_t& k1) {
    k0 = 0; k1 = 0;
    for (uint32_t i = 0; i < len && i < 8; ++i) k0 |= static_cast<uint64_t>(bytes[i]) << (8 * i);
    for (uint32_t i = 8; i < len; ++i) k1 |= static_cast<uint64_t>(bytes[i]) << (8 * (i - 8));
    k1 |= static_cast<uint64_t>(len) << 56;
}

// Longest added-token literal the kernels' halo can see (see encode_kernels.cu).
constexpr uint32_t kMaxAddedBytes = 96;

}  // namespace gtok
