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
    uint32_t family = 0, ignore_merges = 0, monotone = 1, added_ws = 0;
};

// Returns false (with a reason) when a table cannot be built within its probe
// limit or an added-token literal is too long for the on-device matcher.
bool build_host_tables(const HostVocab& hv, HostTables& out, std::string& err);

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
