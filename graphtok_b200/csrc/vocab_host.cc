// tokenizer.json -> HostVocab.  See vocab_host.h for the contract.
#include "vocab_host.h"
#include "json_min.h"

#include <algorithm>
#include <cstdio>
#include <fstream>
#include <map>
#include <sstream>
#include <unordered_map>

namespace gtok {

namespace {

// The exact Split patterns of the two regex-driven families
// (reference: src/vocab.cc:124-131).  GPT-2's pattern is built into the
// ByteLevel pre-tokenizer and never appears in the file.
const char* const kLlama3Pattern =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|"
    "\\p{N}{1,3}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|"
    "\\s+(?!\\S)|\\s+";
const char* const kQwen25Pattern =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|"
    "\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|"
    "\\s+(?!\\S)|\\s+";

// DeepSeek-V3: three Split steps (reference: src/vocab.cc:132-137).  The carriage return and the
// line feed of the main pattern are the characters themselves, as the JSON file's \r and \n
// escapes decode.
const char* const kDeepSeekDigitPattern = "\\p{N}{1,3}";
const char* const kDeepSeekCjkPattern = "[\xe4\xb8\x80-\xe9\xbe\xa5\xe3\x81\x80-\xe3\x82\x9f\xe3\x82\xa0-\xe3\x83\xbf]+";
const char* const kDeepSeekMainPattern =
    "[!\"#$%&'()*+,\\-./:;<=>?@\\[\\\\\\]^_`{|}~][A-Za-z]+|"
    "[^\r\n\\p{L}\\p{P}\\p{S}]?[\\p{L}\\p{M}]+|"
    " ?[\\p{P}\\p{S}]+[\r\n]*|\\s*[\r\n]+|\\s+(?!\\S)|\\s+";

struct ByteMaps {
    uint32_t b2u[256];
    int u2b[0x200];
    ByteMaps() {
        for (int& x : u2b) x = -1;
        bool printable[256] = {};
        for (int b = 0x21; b <= 0x7E; ++b) printable[b] = true;
        for (int b = 0xA1; b <= 0xAC; ++b) printable[b] = true;
        for (int b = 0xAE; b <= 0xFF; ++b) printable[b] = true;
        uint32_t extra = 0;
        for (int b = 0; b < 256; ++b) b2u[b] = printable[b] ? static_cast<uint32_t>(b) : 256u + extra++;
        for (int b = 0; b < 256; ++b) u2b[b2u[b]] = b;
    }
};
const ByteMaps& maps() { static const ByteMaps m; return m; }

using json::Value;

bool str_is(const Value* obj, const char* key, const char* want) {
    if (!obj) return false;
    const Value* v = obj->find(key);
    return v && v->is_string() && v->str == want;
}
// Field equals `want`; an absent field counts as `dflt`.
bool bool_is(const Value* obj, const char* key, bool want, bool dflt) {
    const Value* v = obj ? obj->find(key) : nullptr;
    if (!v) return dflt == want;
    return v->is_bool() && v->b == want;
}
bool null_or_absent(const Value* obj, const char* key) {
    const Value* v = obj->find(key);
    return !v || v->is_null();
}
bool empty_or_absent(const Value* obj, const char* key) {
    const Value* v = obj->find(key);
    return !v || v->is_null() || (v->is_string() && v->str.empty());
}
bool is_split(const Value& step, const char* pattern) {
    if (!step.is_object() || !str_is(&step, "type", "Split") || !str_is(&step, "behavior", "Isolated") ||
        !bool_is(&step, "invert", false, false))
        return false;
    const Value* pat = step.find("pattern");
    return pat && pat->is_object() && str_is(pat, "Regex", pattern);
}
bool is_bytelevel(const Value& step, bool trim_offsets, bool use_regex) {
    return step.is_object() && str_is(&step, "type", "ByteLevel") &&
           bool_is(&step, "add_prefix_space", false, false) &&
           bool_is(&step, "trim_offsets", trim_offsets, true) &&
           bool_is(&step, "use_regex", use_regex, true);
}

// Token string in the byte-level alphabet -> raw bytes.  A codepoint outside
// the 256-entry alphabet contributes its low byte, as the reference does
// (src/vocab.cc:103-109).
std::string decode_token(const std::string& s) {
    std::string out;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    size_t n = s.size(), i = 0;
    while (i < n) {
        uint32_t cp;
        size_t adv;
        unsigned char c = p[i];
        if (c < 0x80) { cp = c; adv = 1; }
        else if ((c & 0xE0) == 0xC0 && i + 1 < n) { cp = ((c & 0x1Fu) << 6) | (p[i + 1] & 0x3Fu); adv = 2; }
        else if ((c & 0xF0) == 0xE0 && i + 2 < n) { cp = ((c & 0x0Fu) << 12) | ((p[i + 1] & 0x3Fu) << 6) | (p[i + 2] & 0x3Fu); adv = 3; }
        else if ((c & 0xF8) == 0xF0 && i + 3 < n) {
            cp = ((c & 0x07u) << 18) | ((p[i + 1] & 0x3Fu) << 12) | ((p[i + 2] & 0x3Fu) << 6) | (p[i + 3] & 0x3Fu);
            adv = 4;
        } else { cp = c; adv = 1; }
        int b = unicode_to_byte(cp);
        out.push_back(static_cast<char>(b >= 0 ? b : static_cast<int>(cp & 0xFF)));
        i += adv;
    }
    return out;
}

// Strict decode of one UTF-8 character at s[i]; 0 when there is none.
size_t utf8_char(const std::string& s, size_t i, uint32_t* cp) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    const size_t n = s.size();
    if (i >= n) return 0;
    const unsigned char c = p[i];
    if (c < 0x80) { *cp = c; return 1; }
    auto cont = [&](size_t k) { return i + k < n && (p[i + k] & 0xC0) == 0x80; };
    if (c >= 0xC2 && c <= 0xDF && cont(1)) { *cp = ((c & 0x1Fu) << 6) | (p[i + 1] & 0x3Fu); return 2; }
    if ((c & 0xF0) == 0xE0 && cont(1) && cont(2)) {
        *cp = ((c & 0x0Fu) << 12) | ((p[i + 1] & 0x3Fu) << 6) | (p[i + 2] & 0x3Fu);
        return (*cp >= 0x800 && !(*cp >= 0xD800 && *cp <= 0xDFFF)) ? 3 : 0;
    }
    if (c >= 0xF0 && c <= 0xF4 && cont(1) && cont(2) && cont(3)) {
        *cp = ((c & 0x07u) << 18) | ((p[i + 1] & 0x3Fu) << 12) | ((p[i + 2] & 0x3Fu) << 6) | (p[i + 3] & 0x3Fu);
        return (*cp >= 0x10000 && *cp <= 0x10FFFF) ? 4 : 0;
    }
    return 0;
}
const char* const kBar = "\xe2\x96\x81";      // U+2581, what the Gemma-3 normaliser writes for a space

// Gemma-3 shape: a token string is raw UTF-8.  What it decodes to: U+2581 as a space, "<0xNN>" as that byte.
// fallback_byte: 0..255 for a "<0xNN>" token, else -1.
std::string decode_sp_token(const std::string& s, int* fallback_byte) {
    *fallback_byte = -1;
    if (s.size() == 6 && s[0] == '<' && s[1] == '0' && s[2] == 'x' && s[5] == '>') {
        auto hex = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1; };
        const int h = hex(s[3]), l = hex(s[4]);
        if (h >= 0 && l >= 0) { *fallback_byte = h * 16 + l; return std::string(1, static_cast<char>(h * 16 + l)); }
    }
    std::string out;
    for (size_t i = 0; i < s.size();) {
        if (s.compare(i, 3, kBar) == 0) { out.push_back(' '); i += 3; }
        else out.push_back(s[i++]);
    }
    return out;
}

std::string utf8_of(uint32_t cp) {
    std::string s;
    if (cp < 0x80) s.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { s.push_back(static_cast<char>(0xC0 | (cp >> 6))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { s.push_back(static_cast<char>(0xE0 | (cp >> 12))); s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else {
        s.push_back(static_cast<char>(0xF0 | (cp >> 18))); s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
        s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
    return s;
}

}  // namespace

const uint32_t* byte_to_unicode() { return maps().b2u; }
int unicode_to_byte(uint32_t cp) { return cp < 0x200 ? maps().u2b[cp] : -1; }

const char* family_name(Family f) {
    switch (f) {
        case Family::GPT2: return "GPT2";
        case Family::Llama3: return "Llama3";
        case Family::Qwen25: return "Qwen25";
        case Family::DeepSeekV3: return "DeepSeekV3";
        case Family::Gemma3: return "Gemma3";
    }
    return "?";
}

bool load_tokenizer_json(const std::string& path, HostVocab& out, std::string& err) {
    std::ifstream f(path, std::ios::binary);
    if (!f.is_open()) { err = "cannot open " + path; return false; }
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    Value root;
    {
        json::Parser parser(text.data(), text.size());
        std::string perr;
        if (!parser.parse(root, perr)) { err = "JSON parse error: " + perr; return false; }
    }
    if (!root.is_object()) { err = "top level is not an object"; return false; }
    const Value* model = root.find("model");
    if (!model || !model->is_object()) { err = "top-level 'model' missing"; return false; }
    if (const Value* t = model->find("type")) {
        if (!t->is_string() || t->str != "BPE") { err = "unsupported model.type"; return false; }
    }
    const Value* vocab = model->find("vocab");
    const Value* merges = model->find("merges");
    if (!vocab || !vocab->is_object() || !merges || !merges->is_array()) {
        err = "model.vocab or model.merges missing";
        return false;
    }

    // ---- family by exact structural match -------------------------------
    const Value* norm = root.find("normalizer");
    const Value* pt = root.find("pre_tokenizer");
    const bool norm_null = !norm || norm->is_null();
    bool matched = false;
    out.nfc = false;
    if (pt && norm_null && is_bytelevel(*pt, /*trim_offsets=*/true, /*use_regex=*/true)) {
        out.family = Family::GPT2;
        matched = true;
    } else if (pt && pt->is_object() && str_is(pt, "type", "Sequence")) {
        const Value* seq = pt->find("pretokenizers");
        if (seq && seq->is_array() && seq->arr.size() == 2) {
            if (norm_null && is_split(seq->arr[0], kLlama3Pattern) && is_bytelevel(seq->arr[1], true, false)) {
                out.family = Family::Llama3;
                matched = true;
            } else if (norm && norm->is_object() && str_is(norm, "type", "NFC") &&
                       is_split(seq->arr[0], kQwen25Pattern) && is_bytelevel(seq->arr[1], false, false)) {
                out.family = Family::Qwen25;
                out.nfc = true;
                matched = true;
            }
        } else if (seq && seq->is_array() && seq->arr.size() == 4) {
            // an empty normalizer Sequence, three Splits, ByteLevel without its own regex (src/vocab.cc:256-262)
            const Value* items = norm && norm->is_object() && str_is(norm, "type", "Sequence") ? norm->find("normalizers") : nullptr;
            if (items && items->is_array() && items->arr.empty() && is_split(seq->arr[0], kDeepSeekDigitPattern) &&
                is_split(seq->arr[1], kDeepSeekCjkPattern) && is_split(seq->arr[2], kDeepSeekMainPattern) &&
                is_bytelevel(seq->arr[3], true, false)) {
                out.family = Family::DeepSeekV3;
                matched = true;
            }
        }
    }
    if (!matched && norm && norm->is_object() && str_is(norm, "type", "Replace") && str_is(norm, "content", kBar) && pt && pt->is_object()) {
        // Gemma-3: every space becomes U+2581, then a Split on the (now absent) space (src/vocab.cc:267-281)
        const Value* npat = norm->find("pattern");
        const Value* ppat = pt->find("pattern");
        if (npat && npat->is_object() && str_is(npat, "String", " ") && str_is(pt, "type", "Split") && ppat && ppat->is_object() &&
            str_is(ppat, "String", " ") && str_is(pt, "behavior", "MergedWithPrevious") && bool_is(pt, "invert", false, false)) {
            out.family = Family::Gemma3;
            matched = true;
        }
    }
    if (!matched) {
        err = "unsupported pre_tokenizer/normalizer pipeline (only the exact GPT-2, Llama-3, Qwen2.5, DeepSeek-V3 and Gemma-3 shapes load)";
        return false;
    }
    // ---- model options ---------------------------------------------------
    const bool llama = out.family == Family::Llama3, gemma = out.family == Family::Gemma3;
    if (!null_or_absent(model, "dropout") || !empty_or_absent(model, "continuing_subword_prefix") ||
        !empty_or_absent(model, "end_of_word_suffix") || !bool_is(model, "byte_fallback", gemma, false) ||
        !bool_is(model, "fuse_unk", gemma, false) || !bool_is(model, "ignore_merges", llama, false) ||
        (gemma ? !str_is(model, "unk_token", "<unk>") : !null_or_absent(model, "unk_token"))) {
        err = "unsupported BPE model options for this family";
        return false;
    }
    out.ignore_merges = llama;
    out.sp_synthetic = 0;
    out.sp_chars.clear();
    out.sp_before_bar.clear();

    // ---- vocab -----------------------------------------------------------
    std::unordered_map<std::string, uint32_t> id_of;
    id_of.reserve(vocab->obj.size() * 2);
    out.token_bytes.clear();
    out.token_bytes.resize(vocab->obj.size());
    for (const json::Member& m : vocab->obj) {
        if (!m.second.is_number() || !m.second.is_int || m.second.inum < 0 || m.second.inum > 0x7FFFFFFF) {
            err = "vocab id is not a non-negative integer";
            return false;
        }
        uint32_t id = static_cast<uint32_t>(m.second.inum);
        if (id >= out.token_bytes.size()) {
            if (id > (1u << 24)) { err = "vocab id too large"; return false; }
            out.token_bytes.resize(id + 1);
        }
        if (gemma) {
            int fb = -1;
            // (a token with a literal space in it can never be matched: the normaliser leaves no space in the text)
            out.token_bytes[id] = m.first.find(' ') == std::string::npos ? decode_sp_token(m.first, &fb) : std::string();
            if (fb >= 0) out.sp_fallback[fb] = id + 1;          // + 1: 0 = not seen yet
            uint32_t cp = 0;
            if (fb < 0 && utf8_char(m.first, 0, &cp) == m.first.size() && cp != ' ') out.sp_chars.emplace_back(cp, id);
        } else {
            out.token_bytes[id] = decode_token(m.first);
        }
        id_of[m.first] = id;    // a repeated key keeps its last id, like a JSON object
    }
    std::vector<MergeRule> synthetic;
    if (gemma) {
        // (the ids made up below must lie beyond every id of the file, those of its added tokens included)
        if (const Value* at = root.find("added_tokens"); at && at->is_array())
            for (const Value& t : at->arr) {
                const Value* idv = t.is_object() ? t.find("id") : nullptr;
                if (idv && idv->is_number() && idv->inum >= 0 && idv->inum <= (1 << 24) && static_cast<size_t>(idv->inum) >= out.token_bytes.size())
                    out.token_bytes.resize(static_cast<size_t>(idv->inum) + 1);
            }
        for (int b = 0; b < 256; ++b) {
            if (!out.sp_fallback[b]) {
                char buf[64];
                std::snprintf(buf, sizeof buf, "missing byte-fallback token <0x%02X>", b);
                err = buf;
                return false;
            }
            --out.sp_fallback[b];
        }
        std::sort(out.sp_chars.begin(), out.sp_chars.end());
        uint32_t bar_id = 0xFFFFFFFFu;
        for (const auto& c : out.sp_chars) if (c.first == 0x2581u) bar_id = c.second;
        if (bar_id == 0xFFFFFFFFu) { err = "the vocabulary has no token for U+2581"; return false; }
        out.sp_chars.emplace_back(0x20u, bar_id);
        std::sort(out.sp_chars.begin(), out.sp_chars.end());
        for (int b = 0; b < 256; ++b) out.byte_to_id[b] = out.sp_fallback[b];
        // every character of the vocabulary from its bytes: (b0, b1) -> partial, (partial, b2) -> ... -> the character's id
        std::map<std::pair<uint32_t, uint32_t>, uint32_t> made;
        for (const auto& c : out.sp_chars) {
            if (c.first < 0x80) { out.byte_to_id[c.first] = c.second; continue; }
            const std::string bytes = utf8_of(c.first);
            uint32_t cur = out.sp_fallback[static_cast<unsigned char>(bytes[0])];
            for (size_t k = 1; k < bytes.size(); ++k) {
                const uint32_t nxt = out.sp_fallback[static_cast<unsigned char>(bytes[k])];
                const bool last = k + 1 == bytes.size();
                auto it = made.find({cur, nxt});
                if (it == made.end()) {
                    uint32_t res = c.second;
                    if (!last) { res = static_cast<uint32_t>(out.token_bytes.size()); out.token_bytes.push_back(bytes.substr(0, k + 1)); }
                    synthetic.push_back({cur, nxt, res});
                    it = made.emplace(std::make_pair(cur, nxt), res).first;
                }
                cur = it->second;
            }
        }
    }
    for (int b = 0; b < 256 && !gemma; ++b) {
        auto it = id_of.find(utf8_of(byte_to_unicode()[b]));
        if (it == id_of.end()) {
            char buf[64];
            std::snprintf(buf, sizeof buf, "missing single-byte token for byte 0x%02x", b);
            err = buf;
            return false;
        }
        out.byte_to_id[b] = it->second;
    }

    // ---- merges ----------------------------------------------------------
    out.merges.clear();
    out.merges.reserve(merges->arr.size());
    if (merges->arr.size() >= (1u << 26)) { err = "more than 2^26 merges"; return false; }
    for (const Value& m : merges->arr) {
        std::string l, r;
        if (m.is_string()) {
            size_t sp = m.str.find(' ');
            if (sp == std::string::npos) { err = "malformed merge entry"; return false; }
            l = m.str.substr(0, sp);
            r = m.str.substr(sp + 1);
        } else if (m.is_array() && m.arr.size() == 2 && m.arr[0].is_string() && m.arr[1].is_string()) {
            l = m.arr[0].str;
            r = m.arr[1].str;
        } else {
            err = "unexpected merge entry type";
            return false;
        }
        auto li = id_of.find(l), ri = id_of.find(r);
        if (li == id_of.end() || ri == id_of.end()) { err = "merge references unknown token"; return false; }
        auto ci = id_of.find(l + r);
        if (ci == id_of.end()) { err = "merge product missing from vocab"; return false; }
        out.merges.push_back({li->second, ri->second, ci->second});
        if (gemma && r.compare(0, 3, kBar) == 0) {
            // the character this rule's left side ends with may be joined to a U+2581 after it: no cut there
            size_t i = l.size();
            while (i > 0 && (static_cast<unsigned char>(l[i - 1]) & 0xC0) == 0x80) --i;
            uint32_t cp = 0;
            if (i > 0 && utf8_char(l, i - 1, &cp)) out.sp_before_bar.push_back(cp == 0x2581u ? 0x20u : cp), out.sp_before_bar.push_back(cp);
        }
    }
    if (gemma) {
        std::sort(out.sp_before_bar.begin(), out.sp_before_bar.end());
        out.sp_before_bar.erase(std::unique(out.sp_before_bar.begin(), out.sp_before_bar.end()), out.sp_before_bar.end());
        out.sp_synthetic = static_cast<uint32_t>(synthetic.size());
        if (synthetic.size() + out.merges.size() >= (1u << 26)) { err = "more than 2^26 merges"; return false; }
        out.merges.insert(out.merges.begin(), synthetic.begin(), synthetic.end());
    }

    // ---- added tokens ----------------------------------------------------
    out.added.clear();
    out.added_max_bytes = 0;
    if (const Value* at = root.find("added_tokens"); at && at->is_array()) {
        std::unordered_map<std::string, uint32_t> seen;
        for (const Value& t : at->arr) {
            if (!t.is_object()) { err = "added token is not an object"; return false; }
            if (!bool_is(&t, "single_word", false, false) || !bool_is(&t, "lstrip", false, false) ||
                !bool_is(&t, "rstrip", false, false)) {
                err = "added token uses unsupported single_word/lstrip/rstrip matching";
                return false;
            }
            const Value* idv = t.find("id");
            const Value* cv = t.find("content");
            uint32_t id = (idv && idv->is_number() && idv->inum >= 0) ? static_cast<uint32_t>(idv->inum) : 0u;
            std::string content = (cv && cv->is_string()) ? cv->str : std::string();
            const Value* nv = t.find("normalized");
            bool normalized = nv && nv->is_bool() && nv->b;
            if (normalized && out.nfc) { err = "normalized added tokens with an NFC normalizer are not supported"; return false; }
            if (content.empty()) continue;
            auto dup = seen.find(content);
            if (dup != seen.end()) {
                if (dup->second != id) { err = "added token content assigned to two ids"; return false; }
                continue;
            }
            seen.emplace(content, id);
            if (id >= out.token_bytes.size()) {
                if (id > (1u << 24)) { err = "added token id too large"; return false; }
                out.token_bytes.resize(static_cast<size_t>(id) + 1);
            }
            if (out.token_bytes[id].empty()) {
                out.token_bytes[id] = content;
            } else {
                // The id already names a model token: its spelling must be this literal.
                bool same = false;
                for (const json::Member& m : vocab->obj)
                    if (static_cast<uint32_t>(m.second.inum) == id && m.first == content) { same = true; break; }
                if (!same) { err = "added token id conflicts with model-vocab content"; return false; }
            }
            if (out.nfc) {
                for (unsigned char c : content)
                    if (c >= 0x80) { err = "non-ASCII added token under an NFC normalizer is not supported"; return false; }
            }
            out.added.push_back({id, content});
            out.added_max_bytes = std::max<uint32_t>(out.added_max_bytes, static_cast<uint32_t>(content.size()));
        }
        // On-device matching looks at each candidate start on its own, which is
        // only sound when no literal contains another literal's first byte
        // after its own first position (reference: src/vocab.cc:812-825).
        bool root_byte[256] = {};
        for (const AddedToken& a : out.added) root_byte[static_cast<unsigned char>(a.content[0])] = true;
        for (const AddedToken& a : out.added)
            for (size_t i = 1; i < a.content.size(); ++i)
                if (root_byte[static_cast<unsigned char>(a.content[i])]) {
                    err = "added-token literals can overlap (a literal contains another literal's first byte)";
                    return false;
                }
    }
    out.vocab_size = static_cast<uint32_t>(out.token_bytes.size());
    if (gemma) {
        // the ids beyond the file's own (partly assembled characters) are not part of the vocabulary
        uint32_t top = 0;
        for (const json::Member& m : vocab->obj) top = std::max(top, static_cast<uint32_t>(m.second.inum) + 1);
        for (const AddedToken& a : out.added) top = std::max(top, a.id + 1);
        out.vocab_size = top;
    }

    // ---- rank monotonicity ------------------------------------------------
    {
        std::vector<uint32_t> last_made(out.token_bytes.size(), 0);   // 1 + highest rank producing the id
        out.monotone = true;
        for (uint32_t k = 0; k < out.merges.size(); ++k)
            last_made[out.merges[k].result] = k + 1;
        for (uint32_t k = 0; k < out.merges.size() && out.monotone; ++k) {
            const MergeRule& m = out.merges[k];
            if (last_made[m.left] > k || last_made[m.right] > k) out.monotone = false;
        }
    }
    return true;
}

}  // namespace gtok
