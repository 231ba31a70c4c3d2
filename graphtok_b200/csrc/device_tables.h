// Layout of the vocabulary tables the encode kernels read.  One definition is
// shared by the host builder (tables_build.cc, which fills plain host vectors)
// and the kernels (which see the same arrays in device memory).
//
// All tables are read-only during an encode and small enough to stay resident
// in the B200's L2 (tens of MB at most): the merge table is 16 B per slot, the
// whole-word table 32 B per slot.
#pragma once
#include <stdint.h>

namespace gtok {

constexpr uint32_t kNoRank = 0xFFFFFFFFu;
constexpr uint32_t kEmptyKey = 0xFFFFFFFFu;
constexpr uint32_t kNoToken = 0xFFFFFFFFu;
constexpr int kWordKeyMax = 15;        // longest pre-token the inline-key word table holds
constexpr int kLitLens = 16;           // distinct added-token literal lengths the hashed matcher takes
constexpr int kProbeLimit = 64;        // every table is built so that no probe chain is longer

// Merge rule table: buckets of two 16-byte slots, one 32-byte memory sector each.  A rule lives in
// its first bucket (merge_buckets) unless that was full when the table was built; only then is it in
// its second bucket, and the first bucket's flag (top bit of `result` in its slot 0, set even when
// that slot is free) says so.  A look-up therefore reads ONE sector, hit or miss, in all but a few
// per cent of the cases: the initial pair probes of the merge kernel are bound by L2 sector
// bandwidth, and a merge step by the latency of its probes.  At least four slots per rule.
//   x = left id, y = right id, z = rank, w = result id (31 bits);  x == kEmptyKey marks a free slot.
// Replaces the reference's Slot64 / Slot128 pair (src/vocab.h:162-201): the
// key and the value arrive in a single 128-bit load.
constexpr uint32_t kBucketSpills = 0x80000000u;   // in slot 0's `result`: some rule of this bucket lives in its second bucket
struct MergeSlot { uint32_t left, right, rank, result; };

// Whole-word table: pre-token bytes (at most 15) -> token id, for pre-tokens whose
// encoding is known to be that single token.  Under ignore_merges (Llama-3) this
// is every vocabulary token, which is the reference's direct table
// (src/vocab.cc:1134-1171); otherwise only tokens whose own bytes merge back to
// themselves, which makes the table a precomputed memo of the merge loop.
//   k0,k1 = bytes 0..7 and 8..15 little-endian, zero padded, with the length in
//   the top byte of k1;  id == kNoToken marks a free slot.
struct WordSlot { uint64_t k0, k1; uint32_t id; uint32_t pad[3]; };

// Long-token table (ignore_merges only): tokens of 16 bytes or more, found by
// a 64-bit hash and confirmed byte for byte against `long_blob`.
struct LongSlot { uint64_t hash; uint32_t id, off, len, pad; };

// Added-token literals by hash (lit_hash_finish of the weighted byte sum, see below);
// id == kNoToken marks a free slot; bytes past the literal's end are zero.
constexpr int kLitInline = 48;
struct alignas(64) LitSlot { uint32_t hash, id, len, pad; uint8_t bytes[kLitInline]; };

// Added-token (special-token) trie, path-compressed.  root[b] is the node after first byte b,
// or kNoToken.  On arriving at node i the bytes blob[skip[i] >> 8 ...] (skip[i] & 0xFF of them)
// must follow in the text (a chain of single-child nodes folded into one, so that the long
// common stems of literals like <|reserved_special_token_N|> cost one node instead of one
// node per byte); then terminal[i] is the token id ending there or kNoToken, and the node
// owns edges [first[i], first[i]+count[i]), sorted by byte; an edge is (next_node << 8) | byte.
struct DeviceTables {
    const MergeSlot* merge;     uint32_t merge_shift;     // buckets of two slots = 2^(32 - merge_shift)
    const WordSlot* word;       uint32_t word_mask;
    const LongSlot* longtab;    uint32_t long_mask;
    const uint8_t* long_blob;   uint32_t long_max_len;
    const uint32_t* byte_to_id;          // [256]
    const uint16_t* uc_stage1;           // unicode class table, see unicode_class_table.h (unicode_wide_table.h when uc_wide)
    const uint32_t* uc_stage2;
    const uint32_t* trie_root;           // [256]
    const uint32_t* trie_first;
    const uint16_t* trie_count;
    const uint32_t* trie_terminal;
    const uint32_t* trie_edges;
    const uint32_t* trie_skip;
    const uint8_t* trie_blob;
    uint32_t added_max_bytes;            // 0 when the vocabulary has no added tokens
    uint32_t lit1_bits[8];               // bytes that open an added-token literal (one bit per byte value)
    uint32_t lit2_bits[8];               // bytes that come second in one
    uint32_t lit_single;                 // some literal is a single byte
    // The literals once more as a hash table keyed by their bytes, each 64-byte slot holding the
    // literal itself, with the distinct literal lengths in ascending order: the longest literal
    // at a position is then found by hashing the text bytes once per pass and reading one slot
    // per literal length, instead of a walk down the trie with a dependent load per step.
    // lit_n_lens == 0 (more than kLitLens distinct lengths, or a literal too long for a slot):
    // only the trie is used.
    const LitSlot* littab;      uint32_t lit_mask;
    uint32_t lit_n_lens;
    uint32_t lit_lens[16];
    uint32_t family;                     // 0 GPT-2, 1 Llama-3, 2 Qwen2.5, 3 DeepSeek-V3, 4 Gemma-3
    uint32_t sp_ascii_known[4];          // Gemma-3: bit c = the ASCII character c is a token of the vocabulary (the space stands for U+2581)
    uint32_t sp_ascii_before_bar[4];     // ... and a rule may join it to a U+2581 after it
    uint32_t uc_wide;                    // the class table is the wide one (unicode_wide_table.h: four bits per codepoint)
    uint32_t ignore_merges;
    uint32_t monotone;
    uint32_t added_ws;                   // some added-token literal contains an ASCII whitespace byte (space, tab, CR, LF, VT, FF)
    uint32_t added_alpha_end;            // some added-token literal ends with an ASCII letter
    uint32_t lit_first, lit_first_n;     // the distinct first bytes of the literals, one per byte of lit_first when there are at most four
    // Normalisation data (nfc_tables.h), uploaded only for vocabularies that declare NFC.
    const uint32_t* nfc_attn_bits;       // one bit per BMP codepoint that can make a text non-NFC
    const uint32_t* nfc_attn_sup;        // (lo, hi) ranges of such codepoints above the BMP
    const uint32_t* nfc_ccc;             // (codepoint, combining class) pairs, ascending
    const uint32_t* nfc_decomp;          // (codepoint, n, d0..d3) full canonical decompositions, ascending
    const uint32_t* nfc_comp;            // (first, second, composite) primary composites, ascending
    uint32_t nfc_attn_sup_n, nfc_ccc_n, nfc_decomp_n, nfc_comp_n;
    uint32_t nfc_lead_quiet[8];          // bit b: no codepoint of nfc_attn_* begins with byte b in UTF-8
    const uint32_t* nfc_cp_hash;         // codepoint -> combining class | (index into nfc_decomp + 1) << 8: (codepoint, that) per slot, codepoint = 0xFFFFFFFF: empty
    uint32_t nfc_cp_hash_mask;
    const uint32_t* nfc_comp_hash;       // nfc_comp as an open-addressed table: (first, second, composite, 0) per slot, first = 0xFFFFFFFF: empty
    uint32_t nfc_comp_hash_mask;
};

// ---- hashes (host and device) ------------------------------------------------
#if defined(__CUDACC__)
#define GTOK_HD __host__ __device__ __forceinline__
#else
#define GTOK_HD inline
#endif

// 32-bit arithmetic only: this sits on the critical path of every merge step.  The two bucket
// numbers are the top bits of two different multiples of one mixed word; `shift` = 32 - log2(buckets).
GTOK_HD void merge_buckets(uint32_t l, uint32_t r, uint32_t shift, uint32_t* b1, uint32_t* b2) {
    uint32_t x = l * 0x9E3779B1u ^ (r + 0x7F4A7C15u) * 0x85EBCA77u;
    x ^= x >> 15;
    *b1 = (x * 0x2C1B3C6Du) >> shift;
    *b2 = *b1 ^ (((x * 0x297A2D39u + 0x68E31DA4u) >> shift) | 1u);      // never the same bucket
}
GTOK_HD uint32_t word_hash(uint64_t k0, uint64_t k1) {
    uint64_t x = k0 * 0x9E3779B185EBCA87ULL + (k1 ^ (k1 >> 29)) * 0xC2B2AE3D27D4EB4FULL;
    x ^= x >> 32; x *= 0xD6E8FEB86659FD93ULL;
    x ^= x >> 32;
    return static_cast<uint32_t>(x);
}
// Hash of a literal: sum of byte j times K^(j+1) (mod 2^32), folded with the length.  A sum, so that
// the hashes of all prefixes of a text come out of one pass, or each from a thread of its own.
constexpr uint32_t kLitHashK = 0x9E3779B1u;
GTOK_HD uint32_t lit_hash_finish(uint32_t h, uint32_t len) {
    uint32_t x = h ^ (len * 0x85EBCA77u);
    x ^= x >> 15; x *= 0x85EBCA6Bu; x ^= x >> 13;
    return x;
}
// FNV-1a over the bytes, folded with the length; used for the long-token table.
GTOK_HD uint32_t nfc_cp_hash(uint32_t cp) { return (cp * 0x9E3779B1u) >> 12; }
GTOK_HD uint32_t nfc_comp_hash(uint32_t first, uint32_t second) { return (first * 0x9E3779B1u) ^ (second * 0x85EBCA6Bu) ^ ((first * 0x9E3779B1u) >> 15); }
GTOK_HD uint64_t long_hash_step(uint64_t h, uint8_t b) { return (h ^ b) * 1099511628211ULL; }
constexpr uint64_t kLongHashSeed = 1469598103934665603ULL;
GTOK_HD uint64_t long_hash_finish(uint64_t h, uint32_t len) {
    h ^= len; h *= 0x9E3779B185EBCA87ULL; h ^= h >> 32;
    return h;
}

}  // namespace gtok
