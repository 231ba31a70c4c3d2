// Host-side vocabulary: what a Hugging Face tokenizer.json says, reduced to the
// pieces the encode path needs.  Pure C++17, no CUDA.
//
// Mirrors the acceptance rules of the reference loader
// (src/vocab.cc:308-618 load_hf_tokenizer_json, :227-306 detect_regex_kind):
// only byte-level BPE files whose normalizer / pre_tokenizer sections have
// exactly the GPT-2, Llama-3, Qwen2.5 or DeepSeek-V3 shape load; everything else is a
// load failure, never a silent approximation.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace gtok {

enum class Family : uint8_t { GPT2 = 0, Llama3 = 1, Qwen25 = 2, DeepSeekV3 = 3 };

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
};

// Loads `path`.  On failure returns false and puts a one-line reason in `err`.
bool load_tokenizer_json(const std::string& path, HostVocab& out, std::string& err);

const char* family_name(Family f);

// GPT-2 byte <-> printable-codepoint map used by byte-level vocabularies.
// byte_to_unicode()[b] is in 0x21..0x143; unicode_to_byte(cp) is -1 if unmapped.
const uint32_t* byte_to_unicode();
int unicode_to_byte(uint32_t cp);

}  // namespace gtok
