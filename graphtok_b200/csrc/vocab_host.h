// Host-side vocabulary: what a Hugging Face tokenizer.json says, reduced to the
// pieces the encode path needs.  Pure C++17, no CUDA.
//
// Mirrors the acceptance rules of the reference loader
// (src/vocab.cc:308-618 load_hf_tokenizer_json, :227-306 detect_regex_kind):
// only byte-level BPE files whose normalizer / pre_tokenizer sections have
// exactly the GPT-2, Llama-3, Qwen2.5 or DeepSeek-V3 shape load, and the Gemma-3 shape (a
// SentencePiece-style BPE over characters with byte fallback, src/vocab.cc:267-281);
// everything else is a load failure, never a silent approximation.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace gtok {

enum class Family : uint8_t { GPT2 = 0, Llama3 = 1, Qwen25 = 2, DeepSeekV3 = 3, Gemma3 = 4 };

struct MergeRule {
    uint32_t left, right, result;   // token ids; the rule's rank is its index
};

struct AddedToken {
    uint32_t id;
    std::string content;            // raw UTF-8 literal matched in the input
};

struct HostVocab {
    Family family = Family::GPT2;
    bool nfc = false;               // normalizer {type: NFC}
    bool ignore_merges = false;     // model.ignore_merges (Llama-3)
    uint32_t vocab_size = 0;        // ids 0 .. vocab_size-1 (incl. added tokens)
    std::vector<std::string> token_bytes;   // id -> raw bytes (empty if unused id)
    uint32_t byte_to_id[256];
    std::vector<MergeRule> merges;  // in rank order
    std::vector<AddedToken> added;
    uint32_t added_max_bytes = 0;
    // True when every rule's operands are byte tokens or results of strictly
    // earlier rules only.  Then a merge never creates a pair of lower rank than
    // itself, which is what lets long pre-tokens be merged one rank at a time
    // over all positions at once.
    bool monotone = true;
    // Gemma-3 shape only.  The model merges characters, not bytes, writes a space as U+2581 and spells a character it
    // does not know as its UTF-8 bytes ("<0xNN>" tokens).  It is brought to the byte-level form the rest of the path
    // works on: token_bytes holds what a token decodes to (U+2581 as a space, "<0xNN>" as that byte); byte_to_id gives
    // a byte its "<0xNN>" id (an ASCII character of the vocabulary its own id, the space U+2581's); and the first
    // sp_synthetic rules of `merges` put every character of the vocabulary together from those bytes, through ids
    // beyond vocab_size that never leave the merge loop (pre-tokenization keeps the bytes of anything that is not a
    // whole character of the vocabulary apart, so that no such rule sees them).
    uint32_t sp_synthetic = 0;
    std::vector<std::pair<uint32_t, uint32_t>> sp_chars;   // (codepoint, id) of the one-character tokens, ascending; U+2581 under U+0020 too
    std::vector<uint32_t> sp_before_bar;                   // codepoints that end the left side of a rule whose right side begins with U+2581, ascending
    uint32_t sp_fallback[256] = {};                        // ids of "<0x00>" .. "<0xFF>"
};

// Loads `path`.  On failure returns false and puts a one-line reason in `err`.
bool load_tokenizer_json(const std::string& path, HostVocab& out, std::string& err);

const char* family_name(Family f);

// GPT-2 byte <-> printable-codepoint map used by byte-level vocabularies.
// byte_to_unicode()[b] is in 0x21..0x143; unicode_to_byte(cp) is -1 if unmapped.
const uint32_t* byte_to_unicode();
int unicode_to_byte(uint32_t cp);

}  // namespace gtok
