// gpu_bpe_tokenize: command-line front end over libgtok with the reference CLI's modes and output
// files (src/main.cc), so that scripts written against the reference's tool keep working:
//
//   --vocab <tokenizer.json> --input <file>            one document; output = flat uint32 ids
//                                                       (src/main.cc:833-842)
//   --vocab <tokenizer.json> --inputs <f1,f2,...>      batch, one graph replay for all files; output =
//                                                       [n_docs:u32][doc_off:u32 x (n_docs+1)][ids:u32]
//                                                       (src/main.cc:531-549)
//   --vocab <tokenizer.json> --benchmark-input-list <file with one path per line>
//                                                       run i encodes input i mod n; output =
//                                                       [n_runs:u32][offsets:u32 x (n_runs+1)][ids:u32]
//                                                       (src/main.cc:397-419)
//   --vocab <tokenizer.json> --decode --input <ids.bin> uint32 ids in, the bytes they spell out
//   [--output <file>] [--runs N] [--warmup N] [--csv]
//
// With --csv one line per run goes to stdout under the reference's headers; the graph time is the
// CUDA-event time of a replay of the staged input (gtok_x_stage / gtok_x_replay), the end-to-end
// time the wall clock around gtok_encode / gtok_encode_batch.  Chat templates, BOS/EOS wrapping
// and NVTX ranges of the reference tool are not part of this build.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/gtok.h"

namespace {

struct Args {
    std::string vocab, input, inputs, list, output = "tokens.bin";
    int runs = 1, warmup = 0;
    bool csv = false, decode = false;
};

bool read_file(const std::string& path, std::string& out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) { std::fprintf(stderr, "cannot read %s\n", path.c_str()); return false; }
    std::ostringstream ss;
    ss << f.rdbuf();
    out = ss.str();
    return true;
}

bool write_file(const std::string& path, const std::vector<std::pair<const void*, size_t>>& parts) {
    std::ofstream o(path, std::ios::binary);
    if (!o) { std::fprintf(stderr, "cannot write %s\n", path.c_str()); return false; }
    for (const auto& p : parts) o.write(static_cast<const char*>(p.first), static_cast<std::streamsize>(p.second));
    return static_cast<bool>(o);
}

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    std::string cur;
    for (char c : s) {
        if (c == sep) { if (!cur.empty()) out.push_back(cur); cur.clear(); }
        else if (c != '\r') cur.push_back(c);
    }
    if (!cur.empty()) out.push_back(cur);
    return out;
}

double ms_since(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

int usage(const char* argv0) {
    std::fprintf(stderr,
                 "usage: %s --vocab <tokenizer.json> (--input <file> | --inputs <f1,f2,...> | --benchmark-input-list <file>) "
                 "[--output <file.bin>] [--runs N] [--warmup N] [--csv]\n"
                 "       %s --vocab <tokenizer.json> --decode --input <ids.bin> [--output <file>]\n",
                 argv0, argv0);
    return 2;
}

// One document: ids into `ids`; returns false on failure.
bool encode_one(void* h, const std::string& text, std::vector<uint32_t>& ids) {
    ids.resize(text.size() + 16);
    int32_t n = gtok_encode(h, reinterpret_cast<const uint8_t*>(text.data()), static_cast<uint32_t>(text.size()), ids.data(), static_cast<uint32_t>(ids.size()));
    if (n == -2) {                       // text its vocabulary's normaliser lengthens
        ids.resize(3 * text.size() + 64);
        n = gtok_encode(h, reinterpret_cast<const uint8_t*>(text.data()), static_cast<uint32_t>(text.size()), ids.data(), static_cast<uint32_t>(ids.size()));
    }
    if (n < 0) { std::fprintf(stderr, "gtok_encode returned %d: %s\n", n, gtok_x_last_error()); return false; }
    ids.resize(static_cast<size_t>(n));
    return true;
}

float graph_ms(void* h, const std::string& text) {
    float ms = 0.f;
    if (gtok_x_stage(h, reinterpret_cast<const uint8_t*>(text.data()), static_cast<uint32_t>(text.size()), nullptr, 1) < 0) return 0.f;
    if (gtok_x_replay(h, &ms) < 0) return 0.f;
    return ms;
}

}  // namespace

int main(int argc, char** argv) {
    Args a;
    for (int i = 1; i < argc; ++i) {
        const std::string k = argv[i];
        auto next = [&]() -> const char* {
            if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", k.c_str()); std::exit(2); }
            return argv[++i];
        };
        if (k == "--vocab") a.vocab = next();
        else if (k == "--input") a.input = next();
        else if (k == "--inputs") a.inputs = next();
        else if (k == "--benchmark-input-list") a.list = next();
        else if (k == "--output") a.output = next();
        else if (k == "--runs") a.runs = std::atoi(next());
        else if (k == "--warmup") a.warmup = std::atoi(next());
        else if (k == "--csv") a.csv = true;
        else if (k == "--decode") a.decode = true;
        else return usage(argv[0]);
    }
    if (a.vocab.empty() || (!a.input.empty() + !a.inputs.empty() + !a.list.empty()) != 1 || a.runs < 1) return usage(argv[0]);

    // ---- decode: uint32 ids -> bytes ----
    if (a.decode) {
        std::string raw;
        if (a.input.empty() || !read_file(a.input, raw)) return 1;
        void* h = gtok_create(a.vocab.c_str(), 4096);
        if (!h) { std::fprintf(stderr, "gtok_create failed: %s\n", gtok_x_last_error()); return 1; }
        const uint32_t n = static_cast<uint32_t>(raw.size() / 4);
        uint64_t need = 0;
        gtok_x_decode(h, reinterpret_cast<const uint32_t*>(raw.data()), n, nullptr, 0, &need, nullptr);
        std::vector<uint8_t> out(need + 16);
        const int64_t got = gtok_x_decode(h, reinterpret_cast<const uint32_t*>(raw.data()), n, out.data(), out.size(), &need, nullptr);
        if (got < 0) { std::fprintf(stderr, "gtok_x_decode returned %lld: %s\n", static_cast<long long>(got), gtok_x_last_error()); gtok_destroy(h); return 1; }
        const bool ok = write_file(a.output, {{out.data(), static_cast<size_t>(got)}});
        std::fprintf(stderr, "[main] decoded %u ids to %lld bytes in %s\n", n, static_cast<long long>(got), a.output.c_str());
        gtok_destroy(h);
        return ok ? 0 : 1;
    }

    // ---- inputs ----
    std::vector<std::string> paths;
    if (!a.input.empty()) paths.push_back(a.input);
    else if (!a.inputs.empty()) paths = split(a.inputs, ',');
    else {
        std::string listing;
        if (!read_file(a.list, listing)) return 1;
        paths = split(listing, '\n');
    }
    if (paths.empty()) { std::fprintf(stderr, "no input files\n"); return 1; }
    std::vector<std::string> texts(paths.size());
    size_t total = 0, longest = 0;
    for (size_t i = 0; i < paths.size(); ++i) {
        if (!read_file(paths[i], texts[i])) return 1;
        total += texts[i].size();
        longest = std::max(longest, texts[i].size());
    }
    const size_t cap = (!a.inputs.empty() ? total : longest) * 3 + 4096;
    if (cap > 0xFFFFFF00ull) { std::fprintf(stderr, "input too large\n"); return 1; }
    void* h = gtok_create(a.vocab.c_str(), static_cast<uint32_t>(cap));
    if (!h) { std::fprintf(stderr, "gtok_create failed: %s\n", gtok_x_last_error()); return 1; }
    int rc = 0;

    if (!a.inputs.empty()) {
        // ---- batch: one replay for all files ----
        std::string blob;
        std::vector<uint32_t> offs(1, 0);
        for (const std::string& t : texts) { blob += t; offs.push_back(static_cast<uint32_t>(blob.size())); }
        std::vector<uint32_t> tokens(3 * blob.size() + 64), doc_off(texts.size() + 1, 0);
        int32_t n = 0;
        if (a.csv) std::printf("run,n_docs,n_tokens_out,kernel_ms,e2e_ms\n");
        for (int i = -a.warmup; i < a.runs && rc == 0; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            n = gtok_encode_batch(h, reinterpret_cast<const uint8_t*>(blob.data()), offs.data(), static_cast<uint32_t>(texts.size()), tokens.data(),
                                  static_cast<uint32_t>(tokens.size()), doc_off.data());
            const double e2e = ms_since(t0);
            if (n < 0) { std::fprintf(stderr, "gtok_encode_batch returned %d: %s\n", n, gtok_x_last_error()); rc = 1; break; }
            if (i < 0) continue;
            float k_ms = 0.f;
            if (gtok_x_stage(h, reinterpret_cast<const uint8_t*>(blob.data()), static_cast<uint32_t>(blob.size()), offs.data(), static_cast<uint32_t>(texts.size())) >= 0)
                gtok_x_replay(h, &k_ms);
            if (a.csv) std::printf("%d,%zu,%d,%.4f,%.4f\n", i, texts.size(), n, k_ms, e2e);
            else std::fprintf(stderr, "[run %2d] docs=%zu tokens=%d  kernel=%.3f ms  e2e=%.3f ms\n", i, texts.size(), n, k_ms, e2e);
        }
        if (rc == 0) {
            const uint32_t n_docs = static_cast<uint32_t>(texts.size());
            if (!write_file(a.output, {{&n_docs, 4}, {doc_off.data(), doc_off.size() * 4}, {tokens.data(), static_cast<size_t>(n) * 4}})) rc = 1;
            else std::fprintf(stderr, "[main] batch wrote n_docs=%u  total_tokens=%d  to %s\n", n_docs, n, a.output.c_str());
        }
    } else if (!a.list.empty()) {
        // ---- benchmark list: run i encodes input i mod n, every run's ids are kept ----
        std::vector<uint32_t> flat, offsets(1, 0), ids;
        for (int i = 0; i < a.warmup && rc == 0; ++i) if (!encode_one(h, texts[static_cast<size_t>(i) % texts.size()], ids)) rc = 1;
        if (a.csv) std::printf("run,input_index,raw_bytes,backend_bytes,n_tokens_out,kernel_ms,backend_e2e_ms,full_e2e_ms\n");
        for (int i = 0; i < a.runs && rc == 0; ++i) {
            const size_t index = static_cast<size_t>(i) % texts.size();
            const auto t0 = std::chrono::steady_clock::now();
            if (!encode_one(h, texts[index], ids)) { rc = 1; break; }
            const double e2e = ms_since(t0);
            const float k_ms = graph_ms(h, texts[index]);
            flat.insert(flat.end(), ids.begin(), ids.end());
            offsets.push_back(static_cast<uint32_t>(flat.size()));
            if (a.csv) std::printf("%d,%zu,%zu,%zu,%zu,%.4f,%.4f,%.4f\n", i, index, texts[index].size(), texts[index].size(), ids.size(), k_ms, e2e, e2e);
            else std::fprintf(stderr, "[run %2d] input=%zu raw_bytes=%zu backend_bytes=%zu tokens=%zu graph=%.3f ms e2e=%.3f ms full_e2e=%.3f ms\n", i, index,
                              texts[index].size(), texts[index].size(), ids.size(), k_ms, e2e, e2e);
        }
        if (rc == 0) {
            const uint32_t n_runs = static_cast<uint32_t>(a.runs);
            if (!write_file(a.output, {{&n_runs, 4}, {offsets.data(), offsets.size() * 4}, {flat.data(), flat.size() * 4}})) rc = 1;
            else std::fprintf(stderr, "[main] benchmark wrote %d output stream(s), %zu total tokens to %s\n", a.runs, flat.size(), a.output.c_str());
        }
    } else {
        // ---- one document ----
        std::vector<uint32_t> ids;
        for (int i = 0; i < a.warmup && rc == 0; ++i) if (!encode_one(h, texts[0], ids)) rc = 1;
        if (a.csv) std::printf("run,n_tokens_out,n_pretokens,pretok_ms,kernel_ms,e2e_ms,full_e2e_ms\n");
        for (int i = 0; i < a.runs && rc == 0; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            if (!encode_one(h, texts[0], ids)) { rc = 1; break; }
            const double e2e = ms_since(t0);
            const float k_ms = graph_ms(h, texts[0]);
            uint64_t work[6] = {0, 0, 0, 0, 0, 0};
            gtok_x_work_stats(h, work);
            if (a.csv) std::printf("%d,%zu,%llu,%.4f,%.4f,%.4f,%.4f\n", i, ids.size(), static_cast<unsigned long long>(work[0]), 0.0, k_ms, e2e, e2e);
            else std::fprintf(stderr, "[run %2d] tokens=%zu  kernel=%.3f ms  e2e=%.3f ms  full_e2e=%.3f ms\n", i, ids.size(), k_ms, e2e, e2e);
        }
        if (rc == 0) {
            if (!write_file(a.output, {{ids.data(), ids.size() * 4}})) rc = 1;
            else std::fprintf(stderr, "[main] wrote %zu tokens (%zu bytes) to %s\n", ids.size(), ids.size() * 4, a.output.c_str());
        }
    }
    gtok_destroy(h);
    return rc;
}
