// Unicode Normalization Form C on the host, for vocabularies whose tokenizer.json
// declares {"type": "NFC"} (Qwen2.5).  Plays the role of the reference's host
// normaliser (src/vocab.cc:1234-1668, normalize_view_for_vocab): a quick scan that leaves
// already-normalised text untouched, and re-normalisation of the stretches around the
// codepoints that can make a text non-NFC.  Tables: nfc_tables.h (Unicode 15.0).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace gtok {

// Returns false and leaves `out` untouched when `text` is already NFC (use the input as
// is); otherwise writes the normalised bytes to `out` and returns true.  Bytes that are
// not valid UTF-8 are passed through unchanged and act as barriers.
bool nfc_normalize(const uint8_t* text, size_t len, std::string& out);

// The same tables as flat arrays of 32-bit words, for upload to the device
// (layouts in device_tables.h).
struct NfcWords {
    std::vector<uint32_t> attn_bits, attn_sup, ccc, decomp, comp;
    uint32_t lead_quiet[8];      // bit b: no such codepoint's UTF-8 form begins with byte b
    std::vector<uint32_t> cp_hash;     // codepoint -> (combining class, index into decomp + 1 or 0): open-addressed (codepoint, class | index << 8) slots, codepoint = 0xFFFFFFFF: empty
    std::vector<uint32_t> comp_hash;   // the composites again as an open-addressed table of (first, second, composite, 0) slots; first = 0xFFFFFFFF: empty
};
void nfc_table_words(NfcWords& out);

}  // namespace gtok
