// Seeded synthetic inputs for the encode path: text generators for the five
// benchmark configurations and a greedy BPE trainer that writes a Hugging Face
// tokenizer.json of the GPT-2, Llama-3 or Qwen2.5 shape.  Everything is driven
// by an explicit 64-bit seed and a fixed PRNG, so the same command line gives
// the same bytes on every machine.  These files stand in for the real
// vocabularies and corpora, which are not redistributable with this tree.
//
//   datagen text  <config 0|1|3|4> <seed> <bytes> <out> [--nfc] [--no-specials]
//   datagen batch <seed> <n_docs> <out_blob> <out_offsets_u32>
//   datagen train <gpt2|llama3|qwen25> <corpus> <n_merges> <n_specials> <out.json>
//   datagen split <gpt2|llama3|qwen25> <text> <out_starts_u32>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

#include "seqsplit.h"

namespace {

using gtok_datagen::SplitFamily;

// ---------------------------------------------------------------- PRNG
struct Rng {
    uint64_t s[4];
    explicit Rng(uint64_t seed) {
        uint64_t z = seed + 0x9E3779B97F4A7C15ULL;
        for (auto& x : s) {
            z += 0x9E3779B97F4A7C15ULL;
            uint64_t t = z;
            t = (t ^ (t >> 30)) * 0xBF58476D1CE4E5B9ULL;
            t = (t ^ (t >> 27)) * 0x94D049BB133111EBULL;
            x = t ^ (t >> 31);
        }
    }
    static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
    uint64_t next() {
        uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45);
        return r;
    }
    double unit() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
    uint32_t below(uint32_t n) { return static_cast<uint32_t>((next() >> 32) * static_cast<uint64_t>(n) >> 32); }
    uint32_t range(uint32_t lo, uint32_t hi) { return lo + below(hi - lo + 1); }   // inclusive
};

void put_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) s.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { s.push_back(static_cast<char>(0xC0 | (cp >> 6))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
        s.push_back(static_cast<char>(0xE0 | (cp >> 12))); s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
        s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
        s.push_back(static_cast<char>(0xF0 | (cp >> 18))); s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
        s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
}

// ---------------------------------------------------------------- lexicons
// Fixed (seed-independent) word lists so that a vocabulary trained on one
// seed's corpus fits another seed's document.
struct Zipf {
    std::vector<double> cdf;
    void init(size_t n, double s) {
        cdf.resize(n);
        double acc = 0;
        for (size_t r = 0; r < n; ++r) { acc += 1.0 / std::pow(static_cast<double>(r + 1), s); cdf[r] = acc; }
        for (double& x : cdf) x /= acc;
    }
    size_t draw(Rng& g) const {
        double u = g.unit();
        return static_cast<size_t>(std::lower_bound(cdf.begin(), cdf.end(), u) - cdf.begin());
    }
};

struct Lexicons {
    std::vector<std::string> ascii, cyr, greek;
    std::vector<std::vector<uint32_t>> accented;   // codepoints, composed form
    Zipf z_ascii, z_small;
    Lexicons() {
        Rng g(0x5EED1E81C0DEULL);
        // Letter frequencies roughly English-like so merges have structure.
        const char* pool = "eeeeeeeeeeeetttttttttaaaaaaaaooooooooiiiiiiinnnnnnnsssssshhhhhhrrrrrrddddlllluuucccmmmwwffggyyppbbvkjxqz";
        const size_t pn = std::strlen(pool);
        std::unordered_map<std::string, int> seen;
        while (ascii.size() < 30000) {
            // Lengths 1-12, short words far more common among the frequent ranks.
            uint32_t len = 1 + g.below(12);
            if (ascii.size() < 200) len = 1 + g.below(5);
            std::string w;
            for (uint32_t i = 0; i < len; ++i) w.push_back(pool[g.below(static_cast<uint32_t>(pn))]);
            if (seen.emplace(w, 1).second) ascii.push_back(w);
        }
        auto make2 = [&](std::vector<std::string>& dst, uint32_t lo, uint32_t hi, size_t count) {
            std::unordered_map<std::string, int> s2;
            while (dst.size() < count) {
                uint32_t len = 2 + g.below(9);
                std::string w;
                for (uint32_t i = 0; i < len; ++i) put_utf8(w, g.range(lo, hi));
                if (s2.emplace(w, 1).second) dst.push_back(w);
            }
        };
        make2(cyr, 0x0430, 0x044F, 4000);     // а..я
        make2(greek, 0x03B1, 0x03C9, 2000);   // α..ω
        // Latin-1 accented words: ASCII letters with one to three accented ones.
        const uint32_t acc[] = {0xE0, 0xE1, 0xE2, 0xE3, 0xE4, 0xE5, 0xE7, 0xE8, 0xE9, 0xEA, 0xEB, 0xEC, 0xED, 0xEE,
                                0xEF, 0xF1, 0xF2, 0xF3, 0xF4, 0xF5, 0xF6, 0xF9, 0xFA, 0xFB, 0xFC, 0xFD, 0xFF};
        while (accented.size() < 3000) {
            uint32_t len = 3 + g.below(8);
            std::vector<uint32_t> w;
            uint32_t n_acc = 1 + g.below(3);
            for (uint32_t i = 0; i < len; ++i) w.push_back(static_cast<unsigned char>(pool[g.below(static_cast<uint32_t>(pn))]));
            for (uint32_t k = 0; k < n_acc; ++k) w[g.below(len)] = acc[g.below(sizeof(acc) / sizeof(acc[0]))];
            accented.push_back(w);
        }
        z_ascii.init(ascii.size(), 1.1);
        z_small.init(2000, 1.1);
    }
};

// Canonical decomposition of the Latin-1 accented lower-case letters used above.
bool decompose_latin1(uint32_t cp, uint32_t& base, uint32_t& mark) {
    switch (cp) {
        case 0xE0: base = 'a'; mark = 0x300; return true;  case 0xE1: base = 'a'; mark = 0x301; return true;
        case 0xE2: base = 'a'; mark = 0x302; return true;  case 0xE3: base = 'a'; mark = 0x303; return true;
        case 0xE4: base = 'a'; mark = 0x308; return true;  case 0xE5: base = 'a'; mark = 0x30A; return true;
        case 0xE7: base = 'c'; mark = 0x327; return true;  case 0xE8: base = 'e'; mark = 0x300; return true;
        case 0xE9: base = 'e'; mark = 0x301; return true;  case 0xEA: base = 'e'; mark = 0x302; return true;
        case 0xEB: base = 'e'; mark = 0x308; return true;  case 0xEC: base = 'i'; mark = 0x300; return true;
        case 0xED: base = 'i'; mark = 0x301; return true;  case 0xEE: base = 'i'; mark = 0x302; return true;
        case 0xEF: base = 'i'; mark = 0x308; return true;  case 0xF1: base = 'n'; mark = 0x303; return true;
        case 0xF2: base = 'o'; mark = 0x300; return true;  case 0xF3: base = 'o'; mark = 0x301; return true;
        case 0xF4: base = 'o'; mark = 0x302; return true;  case 0xF5: base = 'o'; mark = 0x303; return true;
        case 0xF6: base = 'o'; mark = 0x308; return true;  case 0xF9: base = 'u'; mark = 0x300; return true;
        case 0xFA: base = 'u'; mark = 0x301; return true;  case 0xFB: base = 'u'; mark = 0x302; return true;
        case 0xFC: base = 'u'; mark = 0x308; return true;  case 0xFD: base = 'y'; mark = 0x301; return true;
        case 0xFF: base = 'y'; mark = 0x308; return true;
        default: return false;
    }
}

// ---------------------------------------------------------------- text
struct TextGen {
    const Lexicons& lx;
    Rng g;
    std::string out;
    size_t col = 0;
    bool nfc_only;
    TextGen(const Lexicons& l, uint64_t seed, bool nfc) : lx(l), g(seed), nfc_only(nfc) {}

    void sep() {   // separator before an item: a space, or a newline about every 80 columns
        if (out.empty()) return;
        if (col >= 72 + g.below(16)) { out.push_back('\n'); col = 0; }
        else { out.push_back(' '); ++col; }
    }
    void emit(const std::string& s) { out += s; col += s.size(); }

    void ascii_item() {
        double u = g.unit();
        if (u < 0.12) {                       // punctuation token, attached to what precedes
            static const char* punct[] = {",", ".", ".", ",", ";", ":", "!", "?", "...", "(", ")", "\"", "'", "-", "--", "'s", "'t", "'re", "'ll", "n't", "/", "=", "==", "->", "{", "}", "[", "]", "#", "&", "*", "+", "%", "$", "@", "_"};
            emit(punct[g.below(sizeof(punct) / sizeof(punct[0]))]);
        } else if (u < 0.15) {                // digit run of 1-6
            sep();
            uint32_t n = 1 + g.below(6);
            std::string d;
            for (uint32_t i = 0; i < n; ++i) d.push_back(static_cast<char>('0' + g.below(10)));
            emit(d);
        } else if (u < 0.17) {                // whitespace run of 2-8
            uint32_t n = 2 + g.below(7);
            for (uint32_t i = 0; i < n; ++i) {
                uint32_t k = g.below(10);
                out.push_back(k < 7 ? ' ' : (k < 8 ? '\t' : '\n'));
            }
            col = 0;
        } else {
            sep();
            std::string w = lx.ascii[lx.z_ascii.draw(g)];
            if (g.unit() < 0.20) w[0] = static_cast<char>(w[0] - 32);
            emit(w);
        }
    }
    void cjk_run() {
        sep();
        uint32_t n = 2 + g.below(19);
        std::string s;
        for (uint32_t i = 0; i < n; ++i) put_utf8(s, 0x4E00 + static_cast<uint32_t>(lx.z_small.draw(g)) * 3 % 5000 + g.below(3));
        emit(s);
    }
    void config1_item() {
        double u = g.unit();
        if (u < 0.85) ascii_item();
        else if (u < 0.95) {
            sep();
            if (g.below(3) != 0) emit(lx.cyr[lx.z_small.draw(g) * 2 % lx.cyr.size()]);
            else emit(lx.greek[lx.z_small.draw(g) % lx.greek.size()]);
        } else if (u < 0.99) cjk_run();
        else { sep(); std::string s; put_utf8(s, 0x1F600 + g.below(80)); emit(s); }
    }
    void code_line() {
        out.push_back('\n'); col = 0;
        uint32_t indent = g.below(4);
        for (uint32_t i = 0; i < indent * 4; ++i) out.push_back(' ');
        static const char* forms[] = {"if (%s == %s) {", "%s = %s(%s);", "return %s[%s];", "for (int %s = 0; %s < %s; ++%s) {",
                                      "}", "%s->%s = &%s;", "// %s %s %s", "def %s(%s, %s):", "%s_%s += 0x%s;", "print(\"%s\", %s)"};
        const char* f = forms[g.below(sizeof(forms) / sizeof(forms[0]))];
        for (const char* p = f; *p; ++p) {
            if (p[0] == '%' && p[1] == 's') {
                std::string w = lx.ascii[lx.z_ascii.draw(g)];
                if (g.below(4) == 0) { w.push_back('_'); w += lx.ascii[lx.z_ascii.draw(g)]; }
                if (g.below(6) == 0) w += std::to_string(g.below(100));
                out += w;
                ++p;
            } else out.push_back(*p);
        }
        out.push_back('\n'); col = 0;
    }
    void config3_item() {
        double u = g.unit();
        if (u < 0.70) ascii_item();
        else if (u < 0.80) {
            sep();
            const std::vector<uint32_t>& w = lx.accented[lx.z_small.draw(g) * 3 % lx.accented.size()];
            bool nfd = !nfc_only && g.below(2) == 0;
            std::string s;
            for (uint32_t cp : w) {
                uint32_t b, m;
                if (nfd && decompose_latin1(cp, b, m)) { put_utf8(s, b); put_utf8(s, m); }
                else put_utf8(s, cp);
            }
            emit(s);
        } else if (u < 0.95) cjk_run();
        else code_line();
    }
    void base64_block() {
        static const char* a = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
        for (int i = 0; i < 4096; ++i) out.push_back(a[g.below(64)]);
    }
    void repeat_block() {
        uint32_t n = 1024 + g.below(64 * 1024 - 1024 + 1);
        static const char* ch = "aexo-=.*z0 \n";
        char c = ch[g.below(12)];
        out.append(n, c);
    }
    void digit_block() {
        uint32_t n = 1 + g.below(10000);
        for (uint32_t i = 0; i < n; ++i) out.push_back(static_cast<char>('0' + g.below(10)));
    }
};

std::string special_name(SplitFamily fam, uint32_t i) {
    char buf[64];
    if (fam == gtok_datagen::kSplitQwen25) std::snprintf(buf, sizeof buf, "<|qwen_special_%u|>", i);
    else if (fam == gtok_datagen::kSplitDeepSeek) std::snprintf(buf, sizeof buf, "<\xef\xbd\x9cspecial\xe2\x96\x81%u\xef\xbd\x9c>", i);   // fullwidth bars, U+2581
    else std::snprintf(buf, sizeof buf, "<|reserved_special_token_%u|>", i);
    return buf;
}

std::string gen_text(int config, uint64_t seed, size_t bytes, bool nfc_only, bool specials) {
    static const Lexicons lx;
    TextGen t(lx, seed, nfc_only);
    t.out.reserve(bytes + 70000);
    if (config == 0) {
        while (t.out.size() < bytes) t.ascii_item();
    } else if (config == 1) {
        while (t.out.size() < bytes) t.config1_item();
    } else if (config == 3) {
        while (t.out.size() < bytes) t.config3_item();
    } else if (config == 4) {
        // Keep each kind's share of the bytes emitted so far near its target.
        const double target[4] = {0.40, 0.30, 0.20, 0.10};
        double got[4] = {0, 0, 0, 0};
        while (t.out.size() < bytes) {
            int k = 0;
            double worst = 1e300;
            double total = got[0] + got[1] + got[2] + got[3] + 1.0;
            for (int i = 0; i < 4; ++i) { double r = got[i] / total - target[i]; if (r < worst) { worst = r; k = i; } }
            size_t before = t.out.size();
            if (k == 0) { size_t want = 2048 + t.g.below(14336); while (t.out.size() - before < want) t.config1_item(); }
            else if (k == 1) t.base64_block();
            else if (k == 2) t.repeat_block();
            else t.digit_block();
            got[k] += static_cast<double>(t.out.size() - before);
            t.out.push_back(t.g.below(2) ? '\n' : ' ');
            t.col = 0;
        }
    } else {
        std::fprintf(stderr, "datagen: unknown text config %d\n", config);
        std::exit(2);
    }
    std::string text = t.out;
    // Cut on a codepoint boundary at or after `bytes`... simply keep whole items.
    if ((config == 1 || config == 4) && specials) {
        // Insert special-token literals at uniformly drawn offsets, moved forward
        // to the next codepoint boundary.
        uint32_t count = config == 1 ? 500 : 500;
        std::vector<size_t> where;
        Rng g2(seed ^ 0xABCDEF1234ULL);
        for (uint32_t i = 0; i < count; ++i) {
            size_t p = static_cast<size_t>(g2.unit() * static_cast<double>(text.size()));
            while (p < text.size() && (static_cast<unsigned char>(text[p]) & 0xC0) == 0x80) ++p;
            where.push_back(p);
        }
        std::sort(where.begin(), where.end());
        std::string with;
        with.reserve(text.size() + count * 32);
        size_t prev = 0;
        for (size_t p : where) {
            with.append(text, prev, p - prev);
            with += special_name(gtok_datagen::kSplitLlama3, g2.below(256));
            prev = p;
        }
        with.append(text, prev, std::string::npos);
        text.swap(with);
    }
    return text;
}

void write_file(const std::string& path, const void* p, size_t n) {
    std::ofstream f(path, std::ios::binary);
    if (!f) { std::fprintf(stderr, "datagen: cannot write %s\n", path.c_str()); std::exit(1); }
    f.write(static_cast<const char*>(p), static_cast<std::streamsize>(n));
}
std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) { std::fprintf(stderr, "datagen: cannot read %s\n", path.c_str()); std::exit(1); }
    return std::string((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

// ---------------------------------------------------------------- trainer
// Byte-level alphabet in the GPT-2 order: the printable bytes first, then the
// remaining ones mapped to U+0100 upward.
struct Alphabet {
    uint32_t id_of_byte[256];
    uint32_t cp_of_byte[256];
    Alphabet() {
        bool printable[256] = {};
        for (int b = 0x21; b <= 0x7E; ++b) printable[b] = true;
        for (int b = 0xA1; b <= 0xAC; ++b) printable[b] = true;
        for (int b = 0xAE; b <= 0xFF; ++b) printable[b] = true;
        uint32_t next_id = 0, extra = 0;
        for (int b = 0; b < 256; ++b) if (printable[b]) { id_of_byte[b] = next_id++; cp_of_byte[b] = static_cast<uint32_t>(b); }
        for (int b = 0; b < 256; ++b) if (!printable[b]) { id_of_byte[b] = next_id++; cp_of_byte[b] = 256 + extra++; }
    }
};

struct Trainer {
    std::vector<std::string> tok;                 // id -> raw bytes
    struct Word { std::vector<uint32_t> sym; int64_t count; };
    std::vector<Word> words;
    std::unordered_map<uint64_t, int64_t> pair_count;
    std::unordered_map<uint64_t, std::vector<uint32_t>> pair_words;
    struct Item { int64_t count; uint64_t pair; };
    struct Less {
        const Trainer* t;
        // Max-heap on count; among equal counts the lexicographically smaller
        // (left bytes, right bytes) pair comes first.
        bool operator()(const Item& a, const Item& b) const {
            if (a.count != b.count) return a.count < b.count;
            const std::string& al = t->tok[a.pair >> 32];
            const std::string& bl = t->tok[b.pair >> 32];
            if (al != bl) return al > bl;
            return t->tok[a.pair & 0xFFFFFFFFu] > t->tok[b.pair & 0xFFFFFFFFu];
        }
    };
    static uint64_t key(uint32_t a, uint32_t b) { return (static_cast<uint64_t>(a) << 32) | b; }

    std::vector<std::pair<uint32_t, uint32_t>> merges;

    void train(const std::unordered_map<std::string, int64_t>& freq, const Alphabet& ab, size_t n_merges) {
        tok.resize(256);
        for (int b = 0; b < 256; ++b) tok[ab.id_of_byte[b]] = std::string(1, static_cast<char>(b));
        // Deterministic word order: sort by bytes.
        std::vector<const std::pair<const std::string, int64_t>*> order;
        order.reserve(freq.size());
        for (const auto& kv : freq) order.push_back(&kv);
        std::sort(order.begin(), order.end(), [](auto* a, auto* b) { return a->first < b->first; });
        words.reserve(order.size());
        for (auto* kv : order) {
            Word w;
            w.count = kv->second;
            for (unsigned char c : kv->first) w.sym.push_back(ab.id_of_byte[c]);
            words.push_back(std::move(w));
        }
        for (uint32_t wi = 0; wi < words.size(); ++wi) {
            const Word& w = words[wi];
            for (size_t i = 0; i + 1 < w.sym.size(); ++i) {
                uint64_t k = key(w.sym[i], w.sym[i + 1]);
                pair_count[k] += w.count;
                std::vector<uint32_t>& v = pair_words[k];
                if (v.empty() || v.back() != wi) v.push_back(wi);
            }
        }
        std::priority_queue<Item, std::vector<Item>, Less> heap(Less{this});
        for (const auto& kv : pair_count) heap.push({kv.second, kv.first});
        while (merges.size() < n_merges && !heap.empty()) {
            Item top = heap.top();
            heap.pop();
            auto it = pair_count.find(top.pair);
            if (it == pair_count.end() || it->second != top.count || top.count <= 0) continue;   // stale
            uint32_t a = static_cast<uint32_t>(top.pair >> 32), b = static_cast<uint32_t>(top.pair);
            uint32_t nid = static_cast<uint32_t>(tok.size());
            tok.push_back(tok[a] + tok[b]);
            merges.emplace_back(a, b);
            std::vector<uint32_t> affected;
            affected.swap(pair_words[top.pair]);
            // Net change per pair over all affected words; only pairs whose
            // count really moved go back on the heap.
            std::vector<std::pair<uint64_t, int64_t>> delta;
            for (uint32_t wi : affected) {
                Word& w = words[wi];
                bool has = false;
                for (size_t i = 0; i + 1 < w.sym.size(); ++i) if (w.sym[i] == a && w.sym[i + 1] == b) { has = true; break; }
                if (!has) continue;
                // Only pairs touching a, b or the new token can change; the rest
                // would cancel out, so they are not recorded at all.
                auto near = [&](uint32_t x) { return x == a || x == b || x == nid; };
                for (size_t i = 0; i + 1 < w.sym.size(); ++i)
                    if (near(w.sym[i]) || near(w.sym[i + 1])) delta.emplace_back(key(w.sym[i], w.sym[i + 1]), -w.count);
                std::vector<uint32_t> ns;
                ns.reserve(w.sym.size());
                for (size_t i = 0; i < w.sym.size();) {
                    if (i + 1 < w.sym.size() && w.sym[i] == a && w.sym[i + 1] == b) { ns.push_back(nid); i += 2; }
                    else { ns.push_back(w.sym[i]); ++i; }
                }
                w.sym.swap(ns);
                for (size_t i = 0; i + 1 < w.sym.size(); ++i) {
                    if (!near(w.sym[i]) && !near(w.sym[i + 1])) continue;
                    uint64_t k = key(w.sym[i], w.sym[i + 1]);
                    delta.emplace_back(k, w.count);
                    if (w.sym[i] == nid || w.sym[i + 1] == nid) {
                        std::vector<uint32_t>& v = pair_words[k];
                        if (v.empty() || v.back() != wi) v.push_back(wi);
                    }
                }
            }
            std::sort(delta.begin(), delta.end());
            for (size_t i = 0; i < delta.size();) {
                uint64_t k = delta[i].first;
                int64_t d = 0;
                for (; i < delta.size() && delta[i].first == k; ++i) d += delta[i].second;
                if (d == 0 || k == top.pair) continue;
                int64_t& c = pair_count[k];
                c += d;
                if (c <= 0) pair_count.erase(k);
                else heap.push({c, k});
            }
            pair_count.erase(top.pair);
        }
    }
};

void json_escape_token(std::string& out, const std::string& bytes, const Alphabet& ab) {
    for (unsigned char c : bytes) {
        uint32_t cp = ab.cp_of_byte[c];
        if (cp == '"') out += "\\\"";
        else if (cp == '\\') out += "\\\\";
        else put_utf8(out, cp);
    }
}

const char* kLlamaRegex =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\\\r\\\\n\\\\p{L}\\\\p{N}]?\\\\p{L}+|\\\\p{N}{1,3}| ?[^\\\\s\\\\p{L}\\\\p{N}]+[\\\\r\\\\n]*|\\\\s*[\\\\r\\\\n]+|\\\\s+(?!\\\\S)|\\\\s+";
const char* kQwenRegex =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\\\r\\\\n\\\\p{L}\\\\p{N}]?\\\\p{L}+|\\\\p{N}| ?[^\\\\s\\\\p{L}\\\\p{N}]+[\\\\r\\\\n]*|\\\\s*[\\\\r\\\\n]+|\\\\s+(?!\\\\S)|\\\\s+";

// The three DeepSeek-V3 patterns as they stand in a tokenizer.json (JSON string escapes applied).
const char* kDeepSeekDigitRegex = "\\\\p{N}{1,3}";
const char* kDeepSeekCjkRegex = "[\xe4\xb8\x80-\xe9\xbe\xa5\xe3\x81\x80-\xe3\x82\x9f\xe3\x82\xa0-\xe3\x83\xbf]+";
const char* kDeepSeekMainRegex =
    "[!\\\"#$%&'()*+,\\\\-./:;<=>?@\\\\[\\\\\\\\\\\\]^_`{|}~][A-Za-z]+|[^\\r\\n\\\\p{L}\\\\p{P}\\\\p{S}]?[\\\\p{L}\\\\p{M}]+| ?[\\\\p{P}\\\\p{S}]+[\\r\\n]*|\\\\s*[\\r\\n]+|\\\\s+(?!\\\\S)|\\\\s+";

int cmd_train(SplitFamily fam, const std::string& corpus_path, size_t n_merges, uint32_t n_specials, const std::string& out_path) {
    std::string corpus = read_file(corpus_path);
    std::vector<uint32_t> starts;
    gtok_datagen::split(reinterpret_cast<const uint8_t*>(corpus.data()), corpus.size(), fam, starts);
    std::unordered_map<std::string, int64_t> freq;
    freq.reserve(1 << 20);
    for (size_t i = 0; i < starts.size(); ++i) {
        size_t e = i + 1 < starts.size() ? starts[i + 1] : corpus.size();
        ++freq[corpus.substr(starts[i], e - starts[i])];
    }
    std::fprintf(stderr, "datagen: %zu pre-tokens, %zu distinct\n", starts.size(), freq.size());
    Alphabet ab;
    Trainer tr;
    tr.train(freq, ab, n_merges);
    if (tr.merges.size() < n_merges)
        std::fprintf(stderr, "datagen: corpus supports only %zu merges (asked for %zu)\n", tr.merges.size(), n_merges);

    std::string j;
    j.reserve(16 << 20);
    j += "{\"version\":\"1.0\",\"truncation\":null,\"padding\":null,\"added_tokens\":[";
    uint32_t base_id = static_cast<uint32_t>(tr.tok.size());
    for (uint32_t i = 0; i < n_specials; ++i) {
        if (i) j += ",";
        j += "{\"id\":" + std::to_string(base_id + i) + ",\"content\":\"" + special_name(fam, i) +
             "\",\"single_word\":false,\"lstrip\":false,\"rstrip\":false,\"normalized\":false,\"special\":true}";
    }
    j += "],";
    if (fam == gtok_datagen::kSplitGPT2) {
        j += "\"normalizer\":null,\"pre_tokenizer\":{\"type\":\"ByteLevel\",\"add_prefix_space\":false,\"trim_offsets\":true,\"use_regex\":true},";
    } else if (fam == gtok_datagen::kSplitLlama3) {
        j += std::string("\"normalizer\":null,\"pre_tokenizer\":{\"type\":\"Sequence\",\"pretokenizers\":[{\"type\":\"Split\",\"pattern\":{\"Regex\":\"") +
             kLlamaRegex + "\"},\"behavior\":\"Isolated\",\"invert\":false},{\"type\":\"ByteLevel\",\"add_prefix_space\":false,\"trim_offsets\":true,\"use_regex\":false}]},";
    } else if (fam == gtok_datagen::kSplitDeepSeek) {
        const std::string split_a = "{\"type\":\"Split\",\"pattern\":{\"Regex\":\"", split_b = "\"},\"behavior\":\"Isolated\",\"invert\":false},";
        j += "\"normalizer\":{\"type\":\"Sequence\",\"normalizers\":[]},\"pre_tokenizer\":{\"type\":\"Sequence\",\"pretokenizers\":[" +
             split_a + kDeepSeekDigitRegex + split_b + split_a + kDeepSeekCjkRegex + split_b + split_a + kDeepSeekMainRegex + split_b +
             "{\"type\":\"ByteLevel\",\"add_prefix_space\":false,\"trim_offsets\":true,\"use_regex\":false}]},";
    } else {
        j += std::string("\"normalizer\":{\"type\":\"NFC\"},\"pre_tokenizer\":{\"type\":\"Sequence\",\"pretokenizers\":[{\"type\":\"Split\",\"pattern\":{\"Regex\":\"") +
             kQwenRegex + "\"},\"behavior\":\"Isolated\",\"invert\":false},{\"type\":\"ByteLevel\",\"add_prefix_space\":false,\"trim_offsets\":false,\"use_regex\":false}]},";
    }
    j += "\"post_processor\":null,\"decoder\":{\"type\":\"ByteLevel\",\"add_prefix_space\":true,\"trim_offsets\":true,\"use_regex\":true},";
    j += "\"model\":{\"type\":\"BPE\",\"dropout\":null,\"unk_token\":null,\"continuing_subword_prefix\":null,\"end_of_word_suffix\":null,"
         "\"fuse_unk\":false,\"byte_fallback\":false,\"ignore_merges\":";
    j += fam == gtok_datagen::kSplitLlama3 ? "true" : "false";
    j += ",\"vocab\":{";
    for (uint32_t id = 0; id < tr.tok.size(); ++id) {
        if (id) j += ",";
        j += "\"";
        json_escape_token(j, tr.tok[id], ab);
        j += "\":" + std::to_string(id);
    }
    j += "},\"merges\":[";
    for (size_t k = 0; k < tr.merges.size(); ++k) {
        if (k) j += ",";
        j += "\"";
        json_escape_token(j, tr.tok[tr.merges[k].first], ab);
        j += " ";
        json_escape_token(j, tr.tok[tr.merges[k].second], ab);
        j += "\"";
    }
    j += "]}}\n";
    write_file(out_path, j.data(), j.size());
    std::fprintf(stderr, "datagen: wrote %s (%zu tokens, %zu merges, %u specials)\n", out_path.c_str(), tr.tok.size(),
                 tr.merges.size(), n_specials);
    return 0;
}

SplitFamily parse_family(const char* s) {
    if (!std::strcmp(s, "gpt2")) return gtok_datagen::kSplitGPT2;
    if (!std::strcmp(s, "llama3")) return gtok_datagen::kSplitLlama3;
    if (!std::strcmp(s, "qwen25")) return gtok_datagen::kSplitQwen25;
    if (!std::strcmp(s, "deepseek")) return gtok_datagen::kSplitDeepSeek;
    std::fprintf(stderr, "datagen: unknown family %s\n", s);
    std::exit(2);
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 6 && !std::strcmp(argv[1], "text")) {
        bool nfc = false, specials = true;
        for (int i = 6; i < argc; ++i) {
            if (!std::strcmp(argv[i], "--nfc")) nfc = true;
            if (!std::strcmp(argv[i], "--no-specials")) specials = false;
        }
        std::string t = gen_text(std::atoi(argv[2]), std::strtoull(argv[3], nullptr, 10), std::strtoull(argv[4], nullptr, 10), nfc, specials);
        write_file(argv[5], t.data(), t.size());
        return 0;
    }
    if (argc == 6 && !std::strcmp(argv[1], "batch")) {
        // Documents of config-0 text; lengths log-normal with median 2 KB and
        // sigma 1.0, clamped to 64 B - 256 KB.
        uint64_t seed = std::strtoull(argv[2], nullptr, 10);
        uint32_t n_docs = static_cast<uint32_t>(std::strtoul(argv[3], nullptr, 10));
        Rng g(seed * 7919 + 17);
        std::string blob;
        std::vector<uint32_t> offs{0};
        for (uint32_t d = 0; d < n_docs; ++d) {
            double u1 = g.unit(), u2 = g.unit();
            double z = std::sqrt(-2.0 * std::log(u1 + 1e-300)) * std::cos(6.283185307179586 * u2);
            double len = 2048.0 * std::exp(1.0 * z);
            size_t want = static_cast<size_t>(std::min(262144.0, std::max(64.0, len)));
            std::string t = gen_text(0, seed * 1000003 + d, want, false, false);
            t.resize(want);   // ASCII only, so any cut is a codepoint boundary
            blob += t;
            offs.push_back(static_cast<uint32_t>(blob.size()));
        }
        write_file(argv[4], blob.data(), blob.size());
        write_file(argv[5], offs.data(), offs.size() * sizeof(uint32_t));
        return 0;
    }
    if (argc == 7 && !std::strcmp(argv[1], "train"))
        return cmd_train(parse_family(argv[2]), argv[3], std::strtoull(argv[4], nullptr, 10),
                         static_cast<uint32_t>(std::strtoul(argv[5], nullptr, 10)), argv[6]);
    if (argc == 5 && !std::strcmp(argv[1], "split")) {
        std::string t = read_file(argv[3]);
        std::vector<uint32_t> starts;
        gtok_datagen::split(reinterpret_cast<const uint8_t*>(t.data()), t.size(), parse_family(argv[2]), starts);
        write_file(argv[4], starts.data(), starts.size() * sizeof(uint32_t));
        return 0;
    }
    std::fprintf(stderr,
                 "usage:\n  datagen text <config 0|1|3|4> <seed> <bytes> <out> [--nfc] [--no-specials]\n"
                 "  datagen batch <seed> <n_docs> <out_blob> <out_offsets_u32>\n"
                 "  datagen train <gpt2|llama3|qwen25> <corpus> <n_merges> <n_specials> <out.json>\n"
                 "  datagen split <gpt2|llama3|qwen25> <text> <out_starts_u32>\n");
    return 2;
}
