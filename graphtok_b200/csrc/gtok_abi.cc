// extern "C" boundary of libgtok.so; see include/gtok.h for the contract.
#include "../../include/gtok.h"

#include <chrono>
#include <condition_variable>
#include <deque>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "device_tables.h"
#include "encode_kernels.h"
#include "engine.h"
#include "shard_plan.h"

namespace {

thread_local std::string g_last_error;

struct Handle {
    std::unique_ptr<gtok::Engine> engine;
    uint32_t cap_bytes = 4096;
    std::vector<uint32_t> rebased;     // scratch for batch offsets
};

// Leader/follower batching (the reference's src/dispatcher.cc:133-205): a request thread
// queues its text; whoever finds no batch in progress becomes the leader, takes everything
// queued so far (up to the byte and document limits), encodes it as ONE batch replay and hands
// each follower its slice.  A request larger than the batch limit runs alone.
struct Request {
    const uint8_t* text;
    uint32_t len;
    uint32_t* out;
    uint32_t max_out;
    int32_t result = 0;
    bool done = false;
};
struct Dispatcher {
    Handle handle;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Request*> queue;
    bool leader_active = false;
    uint32_t max_batch_bytes = 0, max_batch_docs = 0;
    uint64_t stats[5] = {0, 0, 0, 0, 0};
    // leader scratch
    std::vector<uint8_t> blob;
    std::vector<uint32_t> offs, toks, doc_tok;
};

bool open_handle(Handle& h, const char* path, uint32_t max_bytes) {
    if (!path) { g_last_error = "null vocabulary path"; return false; }
    std::string err;
    h.engine.reset(gtok::Engine::create(path, err));
    if (!h.engine) { g_last_error = err; return false; }
    h.cap_bytes = max_bytes < 4096 ? 4096 : max_bytes;
    return true;
}

int32_t do_encode(Handle* h, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out, bool dev) {
    if (!text && len) return -1;
    // A vocabulary's normaliser (NFC for Qwen2.5) runs inside the graph, where the reference
    // runs it on the host before its graph (src/gtok_shim.cc:117-129); as there, the byte cap
    // applies to what comes out of it, so the raw length is not checked here for such vocabularies.
    if (len > h->cap_bytes && (!h->engine->vocab().nfc || len > 3ull * h->cap_bytes)) return -3;   // NFC shrinks a text at most threefold
    int64_t n = h->engine->encode(text, len, h->cap_bytes, out, max_out, dev);
    if (n < 0) g_last_error = h->engine->last_error();
    return static_cast<int32_t>(n);
}

int32_t do_encode_batch(Handle* h, const uint8_t* concat_bytes, const uint32_t* doc_byte_offsets, uint32_t n_docs,
                        uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_offsets, bool dev = false) {
    for (uint32_t i = 0; i < n_docs; ++i)
        if (doc_byte_offsets[i + 1] < doc_byte_offsets[i]) return -1;
    const uint32_t first = doc_byte_offsets[0];
    uint64_t total = static_cast<uint64_t>(doc_byte_offsets[n_docs]) - first;
    const uint32_t* offs = doc_byte_offsets;
    if (total > 0xFFFFFF00ull) return -3;
    if (total > h->cap_bytes && (!h->engine->vocab().nfc || total > 3ull * h->cap_bytes)) return -3;
    if (first != 0) {
        h->rebased.resize(static_cast<size_t>(n_docs) + 1);
        for (uint32_t i = 0; i <= n_docs; ++i) h->rebased[i] = doc_byte_offsets[i] - first;
        offs = h->rebased.data();
    }
    int64_t n = h->engine->encode_batch(concat_bytes + first, offs, n_docs, h->cap_bytes, out_tokens, out_cap, out_doc_offsets, dev);
    if (n < 0) g_last_error = h->engine->last_error();
    return static_cast<int32_t>(n);
}

}  // namespace

extern "C" {

void* gtok_create(const char* vocab_json_path, uint32_t max_bytes) {
    try {
        std::unique_ptr<Handle> h(new Handle());
        if (!open_handle(*h, vocab_json_path, max_bytes)) return nullptr;
        return h.release();
    } catch (const std::exception& e) { g_last_error = e.what(); return nullptr; } catch (...) { return nullptr; }
}

int32_t gtok_encode(void* handle, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out) {
    if (!handle) return -1;
    try { return do_encode(static_cast<Handle*>(handle), text, len, out, max_out, false); } catch (...) { return -1; }
}

int32_t gtok_encode_to_device(void* handle, const uint8_t* text, uint32_t len, void* out_dev, uint32_t max_out) {
    if (!handle || !out_dev) return -1;
    try { return do_encode(static_cast<Handle*>(handle), text, len, static_cast<uint32_t*>(out_dev), max_out, true); } catch (...) { return -1; }
}

int32_t gtok_encode_batch(void* handle, const uint8_t* concat_bytes, const uint32_t* doc_byte_offsets, uint32_t n_docs,
                          uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_offsets) {
    if (!handle || !concat_bytes || !doc_byte_offsets || !out_tokens || !out_doc_offsets || n_docs == 0) return -1;
    try {
        return do_encode_batch(static_cast<Handle*>(handle), concat_bytes, doc_byte_offsets, n_docs, out_tokens, out_cap, out_doc_offsets);
    } catch (...) { return -1; }
}

int32_t gtok_x_encode_batch_to_device(void* handle, const uint8_t* concat_bytes, const uint32_t* doc_byte_offsets, uint32_t n_docs,
                                      void* out_tokens_dev, uint32_t out_cap, void* out_doc_offsets_dev) {
    if (!handle || !concat_bytes || !doc_byte_offsets || !out_tokens_dev || !out_doc_offsets_dev || n_docs == 0) return -1;
    try {
        return do_encode_batch(static_cast<Handle*>(handle), concat_bytes, doc_byte_offsets, n_docs, static_cast<uint32_t*>(out_tokens_dev), out_cap,
                               static_cast<uint32_t*>(out_doc_offsets_dev), true);
    } catch (...) { return -1; }
}

uint32_t gtok_x_set_max_bytes(void* handle, uint32_t max_bytes) {
    if (!handle) return 0;
    Handle* h = static_cast<Handle*>(handle);
    if (max_bytes > h->cap_bytes) h->cap_bytes = max_bytes;
    return h->cap_bytes;
}

uint32_t gtok_cpu_max_bytes(void*) { return 0u; }
void gtok_set_cpu_max_bytes(void*, uint32_t) {}
const char* gtok_cpu_backend(void*) { return "off"; }

void* gtok_dispatcher_create(const char* vocab_json_path, uint32_t /*cpu_workers*/, uint32_t max_batch_bytes,
                             uint32_t max_batch_docs, uint32_t policy) {
    if (!vocab_json_path || policy > 2) return nullptr;
    try {
        std::unique_ptr<Dispatcher> d(new Dispatcher());
        d->max_batch_bytes = max_batch_bytes ? max_batch_bytes : (8u << 20);
        d->max_batch_docs = max_batch_docs ? max_batch_docs : 256;
        if (!open_handle(d->handle, vocab_json_path, d->max_batch_bytes)) return nullptr;
        return d.release();
    } catch (...) { return nullptr; }
}

int32_t gtok_dispatch_encode(void* dispatcher, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out) {
    if (!dispatcher || (!text && len)) return -1;
    try {
        Dispatcher* d = static_cast<Dispatcher*>(dispatcher);
        Request me{text, len, out, max_out};
        std::unique_lock<std::mutex> lock(d->mu);
        d->queue.push_back(&me);
        for (;;) {
            if (me.done) return me.result;
            if (!d->leader_active) break;
            d->cv.wait(lock);
        }
        // Leader: serve batches until this thread's own request has been answered.
        d->leader_active = true;
        while (!me.done) {
            std::vector<Request*> batch;
            uint64_t bytes = 0;
            while (!d->queue.empty() && batch.size() < d->max_batch_docs) {
                Request* r = d->queue.front();
                if (!batch.empty() && bytes + r->len > d->max_batch_bytes) break;
                batch.push_back(r);
                bytes += r->len;
                d->queue.pop_front();
                if (r->len > d->max_batch_bytes) break;        // a large request runs alone
            }
            lock.unlock();
            const auto t0 = std::chrono::steady_clock::now();
            if (bytes > d->handle.cap_bytes) d->handle.cap_bytes = static_cast<uint32_t>(std::min<uint64_t>(bytes, 0xFFFFFFFFull));
            if (batch.size() == 1) {
                Request* r = batch[0];
                r->result = do_encode(&d->handle, r->text, r->len, r->out, r->max_out, false);
            } else {
                d->blob.resize(bytes);
                d->offs.assign(batch.size() + 1, 0);
                uint32_t at = 0;
                for (size_t i = 0; i < batch.size(); ++i) {
                    if (batch[i]->len) std::memcpy(d->blob.data() + at, batch[i]->text, batch[i]->len);
                    at += batch[i]->len;
                    d->offs[i + 1] = at;
                }
                d->toks.resize(bytes * 3 + 64);                  // ids never outnumber normalised bytes, and NFC lengthens a text at most threefold
                d->doc_tok.assign(batch.size() + 1, 0);
                int32_t n = bytes ? do_encode_batch(&d->handle, d->blob.data(), d->offs.data(), static_cast<uint32_t>(batch.size()), d->toks.data(),
                                                    static_cast<uint32_t>(d->toks.size()), d->doc_tok.data())
                                  : 0;
                for (size_t i = 0; i < batch.size(); ++i) {
                    Request* r = batch[i];
                    if (n < 0) { r->result = -1; continue; }
                    uint32_t cnt = d->doc_tok[i + 1] - d->doc_tok[i];
                    if (cnt > r->max_out) { r->result = -2; continue; }
                    if (cnt) std::memcpy(r->out, d->toks.data() + d->doc_tok[i], static_cast<size_t>(cnt) * 4);
                    r->result = static_cast<int32_t>(cnt);
                }
            }
            const uint64_t ns = static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count());
            lock.lock();
            // Counters as the reference keeps them (src/dispatcher.h:48-54): [0] requests answered by a CPU
            // engine (none here: every request runs on the GPU, whatever `policy` and `cpu_workers` say),
            // [1] requests answered from a batch replay, [2] batch replays, [3] requests too large to batch
            // (each ran alone, counted here and not under [1]), [4] nanoseconds spent in replays.
            if (batch.size() == 1 && batch[0]->len > d->max_batch_bytes) d->stats[3] += 1;
            else { d->stats[1] += batch.size(); d->stats[2] += 1; }
            d->stats[4] += ns;
            for (Request* r : batch) r->done = true;
            d->cv.notify_all();
        }
        d->leader_active = false;
        d->cv.notify_all();            // a queued follower takes over as leader
        return me.result;
    } catch (...) { return -1; }
}

void gtok_dispatcher_stats(void* dispatcher, uint64_t* out5) {
    if (!dispatcher || !out5) return;
    Dispatcher* d = static_cast<Dispatcher*>(dispatcher);
    std::lock_guard<std::mutex> lock(d->mu);
    std::memcpy(out5, d->stats, sizeof d->stats);
}

void gtok_dispatcher_destroy(void* dispatcher) { delete static_cast<Dispatcher*>(dispatcher); }

uint32_t gtok_vocab_size(void* handle) { return handle ? static_cast<Handle*>(handle)->engine->vocab_size() : 0u; }

void gtok_destroy(void* handle) { delete static_cast<Handle*>(handle); }

const char* gtok_x_last_error(void) { return g_last_error.c_str(); }

uint32_t gtok_x_family(void* handle) {
    if (!handle) return 0xFFFFFFFFu;
    const gtok::HostVocab& hv = static_cast<Handle*>(handle)->engine->vocab();
    return static_cast<uint32_t>(hv.family) | (hv.nfc ? 0x100u : 0u);
}

int32_t gtok_x_stage(void* handle, const uint8_t* bytes, uint32_t len, const uint32_t* doc_byte_offsets, uint32_t n_docs) {
    if (!handle || (!bytes && len)) return -1;
    try {
        Handle* h = static_cast<Handle*>(handle);
        if (len > h->cap_bytes) return -3;
        int r = h->engine->stage(bytes, len, doc_byte_offsets, n_docs, h->cap_bytes);
        if (r < 0) g_last_error = h->engine->last_error();
        return r;
    } catch (...) { return -1; }
}

int32_t gtok_x_replay(void* handle, float* ms_out) {
    if (!handle) return -1;
    try {
        Handle* h = static_cast<Handle*>(handle);
        int64_t n = h->engine->replay_staged(ms_out);
        if (n < 0) g_last_error = h->engine->last_error();
        return static_cast<int32_t>(n);
    } catch (...) { return -1; }
}

int32_t gtok_x_profile(void* handle, float* ms_out6) {
    float* ms_out3 = ms_out6;
    if (!handle || !ms_out3) return -1;
    try {
        Handle* h = static_cast<Handle*>(handle);
        int64_t n = h->engine->profile_staged(ms_out3);
        if (n < 0) g_last_error = h->engine->last_error();
        return static_cast<int32_t>(n);
    } catch (...) { return -1; }
}

int32_t gtok_x_read_boundaries(void* handle, uint32_t* out_words, uint32_t max_words) {
    if (!handle || !out_words) return -1;
    try { return static_cast<int32_t>(static_cast<Handle*>(handle)->engine->read_boundaries(out_words, max_words)); } catch (...) { return -1; }
}

int32_t gtok_x_read(void* handle, uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_offsets) {
    if (!handle) return -1;
    try { return static_cast<int32_t>(static_cast<Handle*>(handle)->engine->read_staged(out_tokens, out_cap, out_doc_offsets)); } catch (...) { return -1; }
}

void gtok_x_table_bytes(void* handle, uint64_t* out3) {
    if (!handle || !out3) return;
    static_cast<Handle*>(handle)->engine->table_bytes(&out3[0], &out3[1], &out3[2]);
}

int32_t gtok_x_launches_per_replay(void* handle, int32_t batch) {
    if (!handle) return -1;
    return static_cast<Handle*>(handle)->engine->launches_per_replay(batch != 0);
}

int32_t gtok_x_boundaries_noalloc(void* handle, const void* text_dev, uint32_t len, void* out_bits_dev, void* cuda_stream) {
    if (!handle) return -1;
    try {
        Handle* h = static_cast<Handle*>(handle);
        std::string err;
        int r = gtok::boundaries_noalloc(*h->engine->device_tables(), h->engine->device_index(), text_dev, len, out_bits_dev,
                                         static_cast<cudaStream_t>(cuda_stream), err);
        if (r < 0) g_last_error = err;
        return r;
    } catch (...) { return -1; }
}

int32_t gtok_x_phase_clocks(void* handle, uint64_t* out32, int32_t reset) {
    if (!handle || !out32) return -1;
    try { return static_cast<Handle*>(handle)->engine->read_phase_clocks(reinterpret_cast<unsigned long long*>(out32), reset != 0); } catch (...) { return -1; }
}

int32_t gtok_x_work_stats(void* handle, uint64_t* out6) {
    if (!handle || !out6) return -1;
    try { return static_cast<Handle*>(handle)->engine->read_work_stats(out6); } catch (...) { return -1; }
}

int32_t gtok_x_timeline(void* handle, uint64_t* out, uint32_t max_words) {
    if (!handle || !out) return -1;
    try { return static_cast<Handle*>(handle)->engine->read_timeline(reinterpret_cast<unsigned long long*>(out), max_words); } catch (...) { return -1; }
}

int32_t gtok_x_token_bytes(void* handle, uint32_t id, uint8_t* out, uint32_t cap) {
    if (!handle) return -1;
    const gtok::HostVocab& hv = static_cast<Handle*>(handle)->engine->vocab();
    if (id >= hv.token_bytes.size()) return -1;
    const std::string& b = hv.token_bytes[id];
    if (out && cap >= b.size() && !b.empty()) std::memcpy(out, b.data(), b.size());
    return static_cast<int32_t>(b.size());
}

int64_t gtok_x_decode(void* handle, const uint32_t* ids, uint32_t n, uint8_t* out, uint64_t max_out, uint64_t* need_out, float* kernel_ms) {
    if (!handle || (!ids && n) || (!out && max_out)) return -1;
    try {
        Handle* h = static_cast<Handle*>(handle);
        int64_t r = h->engine->decode(ids, n, out, max_out, need_out, kernel_ms);
        if (r < 0) g_last_error = h->engine->last_error();
        return r;
    } catch (const std::exception& e) { g_last_error = e.what(); return -1; } catch (...) { return -1; }
}

int32_t gtok_x_plan_chunks(void* handle, const uint8_t* text, uint64_t len, uint32_t n_parts, uint64_t* out_offsets) {
    if (!handle || (!text && len) || !n_parts || !out_offsets) return -1;
    try {
        std::vector<uint64_t> cuts;
        gtok::plan_chunks(static_cast<Handle*>(handle)->engine->vocab(), text, len, n_parts, cuts);
        std::memcpy(out_offsets, cuts.data(), cuts.size() * sizeof(uint64_t));
        return 0;
    } catch (...) { return -1; }
}

int32_t gtok_x_plan_documents(const uint32_t* doc_byte_offsets, uint32_t n_docs, uint32_t n_parts, uint32_t* out_doc_index) {
    if (!doc_byte_offsets || !n_parts || !out_doc_index) return -1;
    try {
        std::vector<uint32_t> cuts;
        gtok::plan_documents(doc_byte_offsets, n_docs, n_parts, cuts);
        std::memcpy(out_doc_index, cuts.data(), cuts.size() * sizeof(uint32_t));
        return 0;
    } catch (...) { return -1; }
}

}  // extern "C"
