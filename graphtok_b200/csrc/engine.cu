// See engine.h.
#include "engine.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>

#include "encode_core.h"
#include "encode_kernels.h"
#include "nfc_host.h"
#include "tables_build.h"
#include "unicode_class_table.h"
#include "unicode_wide_table.h"

namespace gtok {

namespace {

// Every CUDA call is checked; a failure becomes a message and a false/-1 return,
// never an abort, so that no error crosses the C ABI as anything but a code.
#define GTOK_CUDA(call)                                                                        \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            err = std::string(#call) + ": " + cudaGetErrorString(e_);                          \
            return false;                                                                      \
        }                                                                                      \
    } while (0)

template <class T>
bool upload(const std::vector<T>& v, const T** dst, std::vector<void*>& owned, std::string& err) {
    void* p = nullptr;
    size_t bytes = std::max<size_t>(v.size() * sizeof(T), 16);
    GTOK_CUDA(cudaMalloc(&p, bytes));
    owned.push_back(p);
    if (!v.empty()) GTOK_CUDA(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    *dst = static_cast<const T*>(p);
    return true;
}

// A few host threads that share the staging copies of one call: text into pinned memory and
// ids out of it move at memcpy speed, which one thread cannot keep near what PCIe carries.
// The workers only run the job's function (plain memcpy); every CUDA call stays on the
// calling thread.  start() publishes a job of `parts` pieces, take() hands out the next piece
// (to workers and to the caller alike), finish() returns when all pieces are done.  Workers
// spin for a short while after a job, so that the copy-out of a call finds them awake after
// its copy-in, then sleep on a condition variable.
class CopyPool {
public:
    // spin_us: how long an idle worker keeps polling for the next job before it sleeps
    CopyPool(int workers, int spin_us) : spin_us_(spin_us) {
        for (int i = 0; i < workers; ++i) threads_.emplace_back([this] { loop(); });
    }
    ~CopyPool() {
        stop_.store(true);
        { std::lock_guard<std::mutex> lk(mu_); }
        cv_.notify_all();
        for (std::thread& t : threads_) t.join();
    }
    void start(int parts, const std::function<void(int)>* fn) {
        fn_ = fn;
        parts_ = static_cast<uint32_t>(parts);
        remaining_.store(parts);
        const uint64_t gen = (state_.load() >> 32) + 1;
        state_.store(gen << 32, std::memory_order_release);
        if (sleepers_.load() > 0) { { std::lock_guard<std::mutex> lk(mu_); } cv_.notify_all(); }
    }
    // Next piece of the current job, or -1 when none is left.
    int take() {
        uint64_t s = state_.load(std::memory_order_acquire);
        for (;;) {
            const uint32_t next = static_cast<uint32_t>(s);
            if (next >= parts_) return -1;
            if (state_.compare_exchange_weak(s, s + 1, std::memory_order_acq_rel)) return static_cast<int>(next);
        }
    }
    void done_one() { remaining_.fetch_sub(1, std::memory_order_acq_rel); }
    void finish() {
        while (remaining_.load(std::memory_order_acquire) != 0) cpu_relax();
        state_.store((state_.load() & 0xFFFFFFFF00000000ull) | 0xFFFFFFFFull, std::memory_order_release);   // closed: no piece can be taken any more
        while (active_.load(std::memory_order_acquire) != 0) cpu_relax();
        fn_ = nullptr;
    }
    static void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#else
        std::this_thread::yield();
#endif
    }

private:
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            // wait for a job newer than `seen`: spin briefly, then sleep
            auto t0 = std::chrono::steady_clock::now();
            for (uint32_t spins = 0;; ++spins) {
                if (stop_.load()) return;
                if ((state_.load(std::memory_order_acquire) >> 32) != seen) break;
                cpu_relax();
                if ((spins & 255u) == 255u && std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(spin_us_)) {
                    std::unique_lock<std::mutex> lk(mu_);
                    sleepers_.fetch_add(1);
                    cv_.wait(lk, [&] { return stop_.load() || (state_.load(std::memory_order_acquire) >> 32) != seen; });
                    sleepers_.fetch_sub(1);
                    t0 = std::chrono::steady_clock::now();
                }
            }
            active_.fetch_add(1, std::memory_order_acq_rel);
            seen = state_.load(std::memory_order_acquire) >> 32;
            for (int p; (p = take()) >= 0;) { (*fn_)(p); done_one(); }
            active_.fetch_sub(1, std::memory_order_acq_rel);
        }
    }
    int spin_us_ = 1500;
    std::vector<std::thread> threads_;
    std::mutex mu_;
    std::condition_variable cv_;
    const std::function<void(int)>* fn_ = nullptr;
    uint32_t parts_ = 0;
    std::atomic<uint64_t> state_{0};            // job number << 32 | next piece (0xFFFFFFFF = closed)
    std::atomic<int> remaining_{0}, active_{0}, sleepers_{0};
    std::atomic<bool> stop_{false};
};

constexpr size_t kCopyPart = 512 << 10;      // bytes per staging step: small enough to overlap with the DMA of the one before
constexpr int kCopyEvents = 64;

constexpr size_t kTextPad = kTile + kWin + 256;
constexpr uint32_t kHdrWords = 4;     // meta occupies the first 4 words of the header; offsets follow

struct Ctx {
    uint32_t cap_bytes = 0, cap_docs = 0, n_tiles_cap = 0;
    bool batch = false;
    uint8_t* d_text = nullptr;
    uint32_t* d_hdr = nullptr;
    uint32_t* d_docmask = nullptr;
    uint8_t* d_raw = nullptr;             // vocabularies that declare NFC: text as given, its header and document bits
    uint32_t* d_rawhdr = nullptr;
    uint32_t* d_docmask_raw = nullptr;
    uint32_t *d_bmask = nullptr, *d_amask = nullptr, *d_tile_nb = nullptr;
    unsigned char* d_ctrl = nullptr;
    size_t ctrl_bytes = 0;
    uint32_t *d_gstage = nullptr, *d_grk = nullptr, *d_gnw = nullptr;
    uint32_t *d_stage = nullptr, *d_ovf = nullptr, *d_glong = nullptr;
    unsigned long long* d_gmiss = nullptr;
    unsigned long long* d_gmed = nullptr;
    unsigned long long* d_gmed1 = nullptr;
    uint32_t *d_out = nullptr, *d_doc_tok = nullptr;
    uint32_t *h_status = nullptr, *d_status = nullptr;
    unsigned long long* d_phase = nullptr;
    uint8_t* h_text = nullptr;
    uint32_t* h_hdr = nullptr;
    // short single documents: text, {length, 1} and ids in page-locked host memory the device reaches
    // directly, and a graph of one single-block kernel (tiny_kernel.cu)
    uint8_t* h_tiny_text = nullptr;
    uint32_t* h_tiny_meta = nullptr;
    uint32_t* h_tiny_out = nullptr;
    cudaGraph_t tiny_graph = nullptr;
    cudaGraphExec_t tiny_exec = nullptr;
    uint32_t* h_out = nullptr;
    size_t h_out_words = 0;
    cudaStream_t stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t ev[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t out_ev[kCopyEvents] = {};
    int nfc_blocks = 1;
    int pretok_blocks = 1, words_blocks = 1, miss_blocks = 1, asm_blocks = 1, docmask_blocks = 1;
    size_t mask_words = 0;
    EncodeArgs args;
    uint32_t staged_docs = 0, staged_len = 0;

    ~Ctx() {
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        if (tiny_exec) cudaGraphExecDestroy(tiny_exec);
        if (tiny_graph) cudaGraphDestroy(tiny_graph);
        if (h_tiny_text) cudaFreeHost(h_tiny_text);
        if (h_tiny_meta) cudaFreeHost(h_tiny_meta);
        if (h_tiny_out) cudaFreeHost(h_tiny_out);
        for (cudaEvent_t e : ev) if (e) cudaEventDestroy(e);
        for (cudaEvent_t e : out_ev) if (e) cudaEventDestroy(e);
        if (stream) cudaStreamDestroy(stream);
        cudaFree(d_raw); cudaFree(d_rawhdr); cudaFree(d_docmask_raw);
        cudaFree(d_text); cudaFree(d_hdr); cudaFree(d_docmask); cudaFree(d_bmask); cudaFree(d_amask);
        cudaFree(d_tile_nb); cudaFree(d_ctrl); cudaFree(d_gstage); cudaFree(d_grk); cudaFree(d_gnw);
        cudaFree(d_out); cudaFree(d_doc_tok); cudaFree(d_phase);
        cudaFree(d_stage); cudaFree(d_ovf); cudaFree(d_glong); cudaFree(d_gmiss); cudaFree(d_gmed); cudaFree(d_gmed1);
        if (h_status) cudaFreeHost(h_status);
        if (h_text) cudaFreeHost(h_text);
        if (h_hdr) cudaFreeHost(h_hdr);
        if (h_out) cudaFreeHost(h_out);
    }
};

}  // namespace

// Decoding context (ids -> bytes): its own stream and captured graph (control block reset ->
// decode kernel), apart from the encode contexts, as in the reference
// (src/tokenizer.cu:5225-5232).  Grows on demand.
struct DecCtx {
    uint32_t cap_ids = 0, n_tiles_cap = 0;
    size_t cap_bytes = 0;
    uint32_t* d_in = nullptr;             // [0] = number of ids, ids from word 4 on
    uint8_t* d_out = nullptr;
    unsigned char* d_ctrl = nullptr;
    size_t ctrl_bytes = 0;
    uint32_t *h_status = nullptr, *d_status = nullptr;
    uint32_t* h_in = nullptr;
    uint8_t* h_out = nullptr;
    cudaStream_t stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t ev[2] = {nullptr, nullptr};
    cudaEvent_t out_ev[kCopyEvents] = {};
    DecodeArgs args;

    ~DecCtx() {
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        for (cudaEvent_t e : ev) if (e) cudaEventDestroy(e);
        for (cudaEvent_t e : out_ev) if (e) cudaEventDestroy(e);
        if (stream) cudaStreamDestroy(stream);
        cudaFree(d_in); cudaFree(d_out); cudaFree(d_ctrl);
        if (h_status) cudaFreeHost(h_status);
        if (h_in) cudaFreeHost(h_in);
        if (h_out) cudaFreeHost(h_out);
    }
};

struct Engine::Impl {
    int device = 0;
    int sm_count = 0;
    HostTables ht;
    DeviceTables dt{};
    std::vector<void*> owned;
    std::unique_ptr<Ctx> single, batch;
    std::unique_ptr<DecCtx> dec;
    const uint32_t* d_tok_off = nullptr;  // decoding tables, uploaded at the first decode
    const uint8_t* d_tok_blob = nullptr;
    const uint32_t* d_tok16 = nullptr;
    uint32_t max_tok_len = 0;
    int dec_per_sm = 1;
    Ctx* staged = nullptr;
    int pretok_per_sm = 1, words_per_sm = 1, miss_per_sm = 1, asm_per_sm = 1, nfc_per_sm = 1;
    bool nfc = false;                    // the vocabulary declares NFC: the graph starts with the normalisation kernel
    bool tiny = true;                    // short single documents take the one-kernel graph (GTOK_TINY=0 turns it off)
    uint32_t last_err_bits = 0;
    std::string norm;                    // host normalisation, used only after kErrNfcLong
    std::string norm_doc;
    std::vector<uint32_t> norm_off;
    std::unique_ptr<CopyPool> pool;      // staging copies of large inputs and outputs
    std::unique_ptr<std::atomic<uint8_t>[]> part_done;
    int part_done_n = 0;

    ~Impl() {
        single.reset();
        batch.reset();
        dec.reset();
        for (void* p : owned) cudaFree(p);
    }

    bool upload_tables(std::string& err) {
        std::vector<uint16_t> s1(gtok_uc_stage1_init, gtok_uc_stage1_init + GTOK_UC_STAGE1_LEN);
        std::vector<uint32_t> s2(gtok_uc_stage2_init, gtok_uc_stage2_init + GTOK_UC_STAGE2_LEN);
        if (ht.family == 3) {        // DeepSeek-V3 asks for marks, punctuation and symbols too
            s1.assign(gtok_uw_stage1_init, gtok_uw_stage1_init + GTOK_UW_STAGE1_LEN);
            s2.assign(gtok_uw_stage2_init, gtok_uw_stage2_init + GTOK_UW_STAGE2_LEN);
        }
        if (ht.family == 4) { s1 = ht.sp_stage1; s2 = ht.sp_stage2; }      // Gemma-3 shape: the vocabulary's own characters
        if (!upload(ht.merge, &dt.merge, owned, err) || !upload(ht.word, &dt.word, owned, err) ||
            !upload(ht.longtab, &dt.longtab, owned, err) || !upload(ht.long_blob, &dt.long_blob, owned, err) ||
            !upload(ht.byte_to_id, &dt.byte_to_id, owned, err) || !upload(s1, &dt.uc_stage1, owned, err) ||
            !upload(s2, &dt.uc_stage2, owned, err) || !upload(ht.trie_root, &dt.trie_root, owned, err) ||
            !upload(ht.trie_first, &dt.trie_first, owned, err) || !upload(ht.trie_count, &dt.trie_count, owned, err) ||
            !upload(ht.trie_terminal, &dt.trie_terminal, owned, err) || !upload(ht.trie_edges, &dt.trie_edges, owned, err) ||
            !upload(ht.trie_skip, &dt.trie_skip, owned, err) || !upload(ht.trie_blob, &dt.trie_blob, owned, err) ||
            !upload(ht.littab, &dt.littab, owned, err))
            return false;
        if (nfc) {
            NfcWords w;
            nfc_table_words(w);
            if (!upload(w.attn_bits, &dt.nfc_attn_bits, owned, err) || !upload(w.attn_sup, &dt.nfc_attn_sup, owned, err) ||
                !upload(w.ccc, &dt.nfc_ccc, owned, err) || !upload(w.decomp, &dt.nfc_decomp, owned, err) ||
                !upload(w.comp, &dt.nfc_comp, owned, err) || !upload(w.comp_hash, &dt.nfc_comp_hash, owned, err) ||
                !upload(w.cp_hash, &dt.nfc_cp_hash, owned, err))
                return false;
            dt.nfc_cp_hash_mask = static_cast<uint32_t>(w.cp_hash.size() / 2 - 1);
            dt.nfc_comp_hash_mask = static_cast<uint32_t>(w.comp_hash.size() / 4 - 1);
            dt.nfc_attn_sup_n = static_cast<uint32_t>(w.attn_sup.size() / 2);
            dt.nfc_ccc_n = static_cast<uint32_t>(w.ccc.size() / 2);
            dt.nfc_decomp_n = static_cast<uint32_t>(w.decomp.size() / 6);
            dt.nfc_comp_n = static_cast<uint32_t>(w.comp.size() / 3);
            for (int i = 0; i < 8; ++i) dt.nfc_lead_quiet[i] = w.lead_quiet[i];
        }
        static_assert(GTOK_UC_STAGE2_LEN == kUcStage2Words && GTOK_UC_STAGE1_LEN >= kUcStage1Bmp, "class table sizes the kernels copy to shared memory");
        fill_table_scalars(ht, dt);
        return true;
    }

    bool upload_decode_tables(const HostVocab& hv, std::string& err) {
        if (d_tok_off) return true;
        std::vector<uint32_t> off(static_cast<size_t>(hv.vocab_size) + 1, 0);
        std::vector<uint8_t> blob;
        std::vector<uint32_t> first16(static_cast<size_t>(hv.vocab_size) * 4 + 4, 0);
        for (uint32_t id = 0; id < hv.vocab_size; ++id) {
            off[id] = static_cast<uint32_t>(blob.size());
            if (id < hv.token_bytes.size()) {
                const std::string& b = hv.token_bytes[id];
                blob.insert(blob.end(), b.begin(), b.end());
                std::memcpy(first16.data() + static_cast<size_t>(id) * 4, b.data(), std::min<size_t>(b.size(), 16));
                max_tok_len = std::max<uint32_t>(max_tok_len, static_cast<uint32_t>(b.size()));
            }
        }
        off[hv.vocab_size] = static_cast<uint32_t>(blob.size());
        if (!upload(blob, &d_tok_blob, owned, err) || !upload(first16, &d_tok16, owned, err)) return false;
        if (!upload(off, &d_tok_off, owned, err)) { d_tok_off = nullptr; return false; }
        dec_per_sm = std::max(1, decode_blocks_per_sm());
        return true;
    }

    bool build_dec(uint32_t cap_ids, size_t cap_bytes, uint32_t vocab_size, std::string& err) {
        std::unique_ptr<DecCtx> c(new DecCtx());
        c->cap_ids = cap_ids;
        c->cap_bytes = cap_bytes;
        c->n_tiles_cap = (cap_ids + kDecIds - 1) / kDecIds + 1;
        GTOK_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        for (cudaEvent_t& e : c->ev) GTOK_CUDA(cudaEventCreate(&e));
        GTOK_CUDA(cudaMalloc(&c->d_in, (static_cast<size_t>(cap_ids) + 4 + kDecPer) * 4));
        GTOK_CUDA(cudaMemset(c->d_in, 0, (static_cast<size_t>(cap_ids) + 4 + kDecPer) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_out, cap_bytes + 16));
        c->ctrl_bytes = 64 + static_cast<size_t>(c->n_tiles_cap + 1) * 8;
        GTOK_CUDA(cudaMalloc(&c->d_ctrl, c->ctrl_bytes));
        GTOK_CUDA(cudaHostAlloc(&c->h_status, 64, cudaHostAllocMapped));
        std::memset(c->h_status, 0, 64);
        GTOK_CUDA(cudaHostGetDevicePointer(&c->d_status, c->h_status, 0));
        GTOK_CUDA(cudaHostAlloc(&c->h_in, (static_cast<size_t>(cap_ids) + 4 + kDecPer) * 4, cudaHostAllocDefault));
        GTOK_CUDA(cudaHostAlloc(&c->h_out, cap_bytes + 16, cudaHostAllocDefault));
        DecodeArgs& a = c->args;
        std::memset(&a, 0, sizeof a);
        a.meta = c->d_in;
        a.ids = c->d_in + 4;
        a.tok_off = d_tok_off;
        a.blob = d_tok_blob;
        a.tok16 = d_tok16;
        a.vocab_size = vocab_size;
        a.ctl = reinterpret_cast<uint32_t*>(c->d_ctrl);
        a.st = reinterpret_cast<unsigned long long*>(c->d_ctrl + 64);
        a.out = c->d_out;
        a.out_cap = static_cast<uint32_t>(std::min<size_t>(cap_bytes, 0xFFFFFFF0u));
        a.status = c->d_status;
        const int blocks = std::max(1, std::min<int>(static_cast<int>(c->n_tiles_cap), sm_count * dec_per_sm));
        GTOK_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        cudaMemsetAsync(c->d_ctrl, 0, c->ctrl_bytes, c->stream);
        launch_decode(a, blocks, c->stream);
        GTOK_CUDA(cudaStreamEndCapture(c->stream, &c->graph));
        GTOK_CUDA(cudaGraphInstantiate(&c->exec, c->graph, 0));
        GTOK_CUDA(cudaGetLastError());
        dec = std::move(c);
        return true;
    }

    bool build_ctx(std::unique_ptr<Ctx>& slot, uint32_t cap_bytes, uint32_t cap_docs, bool batch_mode, std::string& err) {
        std::unique_ptr<Ctx> c(new Ctx());
        c->cap_bytes = cap_bytes;
        c->cap_docs = cap_docs;
        c->batch = batch_mode;
        c->n_tiles_cap = (cap_bytes + kTile - 1) / kTile + 1;
        const size_t tile_bytes = static_cast<size_t>(c->n_tiles_cap) * kTile;
        const size_t mask_words = static_cast<size_t>(c->n_tiles_cap) * kTileWords + 264;
        const size_t hdr_words = kHdrWords + static_cast<size_t>(cap_docs) + 2;
        GTOK_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        for (cudaEvent_t& e : c->ev) GTOK_CUDA(cudaEventCreate(&e));
        GTOK_CUDA(cudaMalloc(&c->d_text, tile_bytes + kTextPad));
        GTOK_CUDA(cudaMemset(c->d_text, 0, tile_bytes + kTextPad));
        GTOK_CUDA(cudaMalloc(&c->d_hdr, hdr_words * 4));
        GTOK_CUDA(cudaMemset(c->d_hdr, 0, hdr_words * 4));
        GTOK_CUDA(cudaMalloc(&c->d_bmask, mask_words * 4));
        GTOK_CUDA(cudaMalloc(&c->d_amask, mask_words * 4));
        GTOK_CUDA(cudaMalloc(&c->d_tile_nb, (c->n_tiles_cap + 1) * 4));
        if (batch_mode) GTOK_CUDA(cudaMalloc(&c->d_docmask, mask_words * 4));
        if (nfc) {
            GTOK_CUDA(cudaMalloc(&c->d_raw, tile_bytes + kTextPad));
            GTOK_CUDA(cudaMemset(c->d_raw, 0, tile_bytes + kTextPad));
            GTOK_CUDA(cudaMalloc(&c->d_rawhdr, hdr_words * 4));
            GTOK_CUDA(cudaMemset(c->d_rawhdr, 0, hdr_words * 4));
            if (batch_mode) GTOK_CUDA(cudaMalloc(&c->d_docmask_raw, mask_words * 4));
        }
        c->ctrl_bytes = 64 + static_cast<size_t>(c->n_tiles_cap + 1) * 28;     // control words, three look-back state arrays, ids per tile
        GTOK_CUDA(cudaMalloc(&c->d_ctrl, c->ctrl_bytes));
        GTOK_CUDA(cudaMemset(c->d_ctrl, 0, c->ctrl_bytes));
        GTOK_CUDA(cudaMalloc(&c->d_gstage, (tile_bytes + 64) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_grk, (tile_bytes + 64) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_gnw, (tile_bytes + 64) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_stage, (tile_bytes + 64) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_ovf, static_cast<size_t>(c->n_tiles_cap) * kTokExtra * 4));
        GTOK_CUDA(cudaMalloc(&c->d_gmiss, (tile_bytes / 2 + 64) * 8));
        GTOK_CUDA(cudaMalloc(&c->d_gmed, (tile_bytes / 16 + 64) * 8));
        GTOK_CUDA(cudaMalloc(&c->d_gmed1, (tile_bytes / 32 + 64) * 8));
        GTOK_CUDA(cudaMalloc(&c->d_glong, static_cast<size_t>(c->n_tiles_cap) * kLongPerTile * 3 * 4));
        GTOK_CUDA(cudaMalloc(&c->d_out, (static_cast<size_t>(cap_bytes) + 16) * 4));
        GTOK_CUDA(cudaMalloc(&c->d_doc_tok, (static_cast<size_t>(cap_docs) + 2) * 4));
        GTOK_CUDA(cudaHostAlloc(&c->h_status, 64, cudaHostAllocMapped));
        std::memset(c->h_status, 0, 64);
        GTOK_CUDA(cudaHostGetDevicePointer(&c->d_status, c->h_status, 0));
        GTOK_CUDA(cudaHostAlloc(&c->h_text, static_cast<size_t>(cap_bytes) + 64, cudaHostAllocDefault));
        GTOK_CUDA(cudaHostAlloc(&c->h_hdr, hdr_words * 4, cudaHostAllocDefault));

        EncodeArgs& a = c->args;
        std::memset(&a, 0, sizeof a);
        a.text = c->d_text;
        a.meta = c->d_hdr;
        a.doc_off = batch_mode ? c->d_hdr + kHdrWords : nullptr;
        a.docmask = batch_mode ? c->d_docmask : nullptr;
        a.bmask = c->d_bmask;
        a.amask = c->d_amask;
        a.tile_nb = c->d_tile_nb;
        a.ctl = reinterpret_cast<uint32_t*>(c->d_ctrl);
        a.st1 = reinterpret_cast<unsigned long long*>(c->d_ctrl + 64);
        a.st2 = a.st1 + (c->n_tiles_cap + 1);
        a.st0 = a.st2 + (c->n_tiles_cap + 1);
        a.tile_tok = reinterpret_cast<uint32_t*>(a.st0 + (c->n_tiles_cap + 1));
        a.sum_tiles = kSumTiles;
        a.text_cap = cap_bytes;
        if (nfc) {
            a.raw = c->d_raw;
            a.raw_meta = c->d_rawhdr;
            a.raw_doc_off = batch_mode ? c->d_rawhdr + kHdrWords : nullptr;
            a.raw_docmask = batch_mode ? c->d_docmask_raw : nullptr;
            a.norm_text = c->d_text;
            a.norm_meta = c->d_hdr;
            a.norm_doc_off = batch_mode ? c->d_hdr + kHdrWords : nullptr;
        }
        a.gstage = c->d_gstage;
        a.gwork_rk = c->d_grk;
        a.gwork_nw = c->d_gnw;
        a.stage = c->d_stage;
        a.ovf = c->d_ovf;
        a.gmiss = c->d_gmiss;
        a.gmed = c->d_gmed;
        a.gmed1 = c->d_gmed1;
        a.gmed_cap = static_cast<uint32_t>(tile_bytes / 16 + 64);
        a.glong_g = c->d_glong;
        a.glong_len = c->d_glong + static_cast<size_t>(c->n_tiles_cap) * kLongPerTile;
        a.glong_cnt = c->d_glong + static_cast<size_t>(c->n_tiles_cap) * kLongPerTile * 2;
        a.out_tokens = c->d_out;
        a.out_cap = cap_bytes + 16;
        a.out_doc_tok = batch_mode ? c->d_doc_tok : nullptr;
        a.status = c->d_status;
        if (std::getenv("GTOK_PHASE_CLOCKS")) {
            GTOK_CUDA(cudaMalloc(&c->d_phase, (kPhaseWords + kTlWords) * sizeof(unsigned long long)));
            GTOK_CUDA(cudaMemset(c->d_phase, 0, (kPhaseWords + kTlWords) * sizeof(unsigned long long)));
            a.phase_clk = c->d_phase;
        }
        a.tb = dt;

        // Capture: control block reset, [document mask], pretok, merge.
        const int pretok_blocks = std::max(1, std::min<int>(static_cast<int>((static_cast<size_t>(cap_bytes) + kPTile - 1) / kPTile), sm_count * pretok_per_sm));
        const int words_blocks = std::max(1, std::min<int>(static_cast<int>(c->n_tiles_cap), sm_count * words_per_sm));
        const int miss_blocks = std::max(1, sm_count * miss_per_sm);
        const int asm_blocks = std::max(1, std::min<int>(static_cast<int>(c->n_tiles_cap), sm_count * asm_per_sm));
        c->pretok_blocks = pretok_blocks;
        c->words_blocks = words_blocks;
        c->miss_blocks = miss_blocks;
        c->asm_blocks = asm_blocks;
        c->nfc_blocks = std::max(1, std::min<int>(static_cast<int>(c->n_tiles_cap), sm_count * nfc_per_sm));
        c->docmask_blocks = std::max(1, std::min<int>(sm_count, static_cast<int>((cap_docs + 256) / 256)));
        c->mask_words = mask_words;
        GTOK_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        cudaMemsetAsync(c->d_ctrl, 0, c->ctrl_bytes, c->stream);
        launch_front(c.get());
        launch_pretok(a, pretok_blocks, c->stream);
        launch_words(a, words_blocks, c->stream);
        launch_miss(a, miss_blocks, c->stream);
        launch_assemble(a, asm_blocks, c->stream);
        GTOK_CUDA(cudaStreamEndCapture(c->stream, &c->graph));
        pin_tables_in_l2(c->graph);
        GTOK_CUDA(cudaGraphInstantiate(&c->exec, c->graph, 0));
        GTOK_CUDA(cudaGetLastError());
        if (!batch_mode && !nfc && tiny) {
            // the one-kernel graph for short inputs: same work buffers, text and ids in mapped host memory
            GTOK_CUDA(cudaHostAlloc(&c->h_tiny_text, kTinyMaxBytes + 64, cudaHostAllocMapped));
            GTOK_CUDA(cudaHostAlloc(&c->h_tiny_meta, 64, cudaHostAllocMapped));
            GTOK_CUDA(cudaHostAlloc(&c->h_tiny_out, (static_cast<size_t>(kTinyMaxBytes) + 16) * 4, cudaHostAllocMapped));
            std::memset(c->h_tiny_text, 0, kTinyMaxBytes + 64);
            std::memset(c->h_tiny_meta, 0, 64);
            uint8_t* d_tt = nullptr;
            uint32_t *d_tm = nullptr, *d_to = nullptr;
            GTOK_CUDA(cudaHostGetDevicePointer(&d_tt, c->h_tiny_text, 0));
            GTOK_CUDA(cudaHostGetDevicePointer(&d_tm, c->h_tiny_meta, 0));
            GTOK_CUDA(cudaHostGetDevicePointer(&d_to, c->h_tiny_out, 0));
            EncodeArgs ta = a;
            ta.out_tokens = d_to;
            ta.out_cap = kTinyMaxBytes + 16;
            ta.one_list = 1;
            // (with diagnostics on, the kernel stamps its stages into row 0 of timeline table 5; the per-phase cycle counters of the tile programs are shared with the four-kernel graph)
            GTOK_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
            launch_tiny(ta, d_tt, d_tm, c->stream);
            GTOK_CUDA(cudaStreamEndCapture(c->stream, &c->tiny_graph));
            GTOK_CUDA(cudaGraphInstantiate(&c->tiny_exec, c->tiny_graph, 0));
            GTOK_CUDA(cudaGetLastError());
        }
        slot = std::move(c);
        return true;
    }

    // A short single document through the one-kernel graph.  Returns the id count, -2 when `out` is too
    // small, or kNoCtx when the call should take the four-kernel path (the kernel gave up on something).
    int64_t run_tiny(Ctx* c, const uint8_t* text, uint32_t len, uint32_t* out, uint32_t max_out, std::string& err) {
        std::memcpy(c->h_tiny_text, text, len);
        std::memset(c->h_tiny_text + len, 0, 16);
        c->h_tiny_meta[0] = len;
        c->h_tiny_meta[1] = 1;
        c->h_status[0] = 0;
        c->h_status[1] = 0;
        c->staged_len = len;
        c->staged_docs = 1;
        last_err_bits = 0;
        cudaError_t e = cudaGraphLaunch(c->tiny_exec, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { err = std::string("short-input graph: ") + cudaGetErrorString(e); return -1; }
        if (reinterpret_cast<volatile uint32_t*>(c->h_status)[1]) return kNoCtx;
        const uint32_t total = reinterpret_cast<volatile uint32_t*>(c->h_status)[0];
        if (total > max_out) { err = "more token ids than the output buffer holds"; return -2; }
        std::memcpy(out, c->h_tiny_out, static_cast<size_t>(total) * 4);
        return total;
    }

    // The two big look-up tables are kept resident in L2 (the reference's tables are "L2-resident" by
    // being small; these are 8-32 MiB each and every replay of a large document would otherwise pull
    // a good part of them from DRAM again): a part of L2 is set aside for persisting lines once per
    // engine, and the graph's words kernel gets an access-policy window over the whole-word table, its
    // miss kernel one over the merge table.  Failure of any of this is not an error: the kernels then
    // simply run without the hint.
    size_t l2_persist_bytes = 0;
    void reserve_l2() {
        int max_persist = 0, max_window = 0;
        if (cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, device) != cudaSuccess) { cudaGetLastError(); return; }
        if (const char* env = std::getenv("GTOK_L2_PERSIST")) { if (std::atoi(env) == 0) return; }
        const size_t want = ht.merge.size() * sizeof(MergeSlot) + ht.word.size() * sizeof(WordSlot);
        const size_t take = std::min<size_t>(want, static_cast<size_t>(max_persist));
        if (!take || !max_window) return;
        if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, take) != cudaSuccess) { cudaGetLastError(); return; }
        l2_persist_bytes = take;
        l2_window_max = static_cast<size_t>(max_window);
    }
    size_t l2_window_max = 0;
    void pin_tables_in_l2(cudaGraph_t graph) {
        if (!l2_persist_bytes) return;
        size_t n = 0;
        if (cudaGraphGetNodes(graph, nullptr, &n) != cudaSuccess || !n) { cudaGetLastError(); return; }
        std::vector<cudaGraphNode_t> nodes(n);
        if (cudaGraphGetNodes(graph, nodes.data(), &n) != cudaSuccess) { cudaGetLastError(); return; }
        const size_t merge_bytes = ht.merge.size() * sizeof(MergeSlot), word_bytes = ht.word.size() * sizeof(WordSlot);
        for (cudaGraphNode_t node : nodes) {
            cudaGraphNodeType type;
            if (cudaGraphNodeGetType(node, &type) != cudaSuccess || type != cudaGraphNodeTypeKernel) continue;
            cudaKernelNodeParams kp;
            if (cudaGraphKernelNodeGetParams(node, &kp) != cudaSuccess) { cudaGetLastError(); continue; }
            const void* base = nullptr;
            size_t bytes = 0;
            if (kp.func == miss_kernel_address()) { base = dt.merge; bytes = merge_bytes; }
            else if (kp.func == words_kernel_address()) { base = dt.word; bytes = word_bytes; }
            if (!base) continue;
            cudaKernelNodeAttrValue v;
            std::memset(&v, 0, sizeof v);
            v.accessPolicyWindow.base_ptr = const_cast<void*>(base);
            v.accessPolicyWindow.num_bytes = std::min(bytes, l2_window_max);
            // the share of the window that fits the set-aside part of L2 persists, the rest streams
            v.accessPolicyWindow.hitRatio = static_cast<float>(std::min(1.0, static_cast<double>(l2_persist_bytes) / static_cast<double>(merge_bytes + word_bytes)));
            v.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
            v.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
            if (cudaGraphKernelNodeSetAttribute(node, cudaKernelNodeAttributeAccessPolicyWindow, &v) != cudaSuccess) cudaGetLastError();
        }
    }

    // Normalisation, in three launches: look for codepoints that can make the raw text non-NFC; if
    // there are none (the usual case) copy text and header over as they are; else normalise.  The
    // second and third each return at once in the case that is not theirs.
    void launch_normalise(Ctx* c) {
        EncodeArgs chk = c->args;
        chk.raw_docmask = nullptr;
        const int wide = std::max(1, std::min<int>(static_cast<int>(c->n_tiles_cap) * 2, sm_count * 8));
        launch_nfc_check(chk, wide, c->stream);
        launch_nfc_copy(c->args, wide, c->stream);
        if (c->batch) {
            cudaMemsetAsync(c->d_docmask_raw, 0, c->mask_words * 4, c->stream);
            launch_raw_docmask(c->args, c->d_docmask_raw, c->docmask_blocks, c->stream);
        }
        launch_nfc(c->args, c->nfc_blocks, c->stream);
    }
    // What precedes pre-tokenization: [normalisation], [document bits].
    void launch_front(Ctx* c) {
        if (nfc) launch_normalise(c);
        if (c->batch) {
            cudaMemsetAsync(c->d_docmask, 0, c->mask_words * 4, c->stream);
            launch_docmask(c->args, c->d_docmask, c->docmask_blocks, c->stream);
        }
    }

    // Context able to take `need_bytes` (and `need_docs`); built or rebuilt on demand.
    Ctx* ctx_for(bool batch_mode, uint32_t need_bytes, uint32_t need_docs, uint32_t cap_hint, std::string& err) {
        std::unique_ptr<Ctx>& slot = batch_mode ? batch : single;
        if (slot && slot->cap_bytes >= need_bytes && slot->cap_docs >= need_docs) return slot.get();
        uint32_t cap = std::max<uint32_t>(std::max<uint32_t>(need_bytes, cap_hint), 4096);
        if (slot) cap = std::max(cap, slot->cap_bytes);
        uint32_t docs = 1;
        if (batch_mode) {
            docs = slot ? slot->cap_docs : 256;
            while (docs < need_docs) {
                if (docs > (0xFFFFFFFFu >> 1)) { err = "document capacity overflow"; return nullptr; }
                docs <<= 1;
            }
        }
        if (staged == slot.get()) staged = nullptr;
        std::unique_ptr<Ctx> fresh;
        if (!build_ctx(fresh, cap, docs, batch_mode, err)) return nullptr;
        slot = std::move(fresh);
        return slot.get();
    }

    bool grow_host_out(Ctx* c, size_t words, std::string& err) {
        if (c->h_out_words >= words) return true;
        if (c->h_out) cudaFreeHost(c->h_out);
        c->h_out = nullptr;
        c->h_out_words = 0;
        size_t want = std::max<size_t>(words, 1 << 16);
        GTOK_CUDA(cudaHostAlloc(&c->h_out, want * 4, cudaHostAllocDefault));
        c->h_out_words = want;
        return true;
    }

    // Host -> pinned -> device.  Large inputs piece by piece through the pool: finished pieces go to
    // the device while the rest is still being copied into pinned memory.
    bool host_to_device(uint8_t* d_dst, uint8_t* h_pin, const uint8_t* src, size_t len, cudaStream_t stream, std::string& err) {
        if (len >= kCopyPart && is_pinned(src)) {
            // the caller's buffer is page-locked: the device reads it directly, no staging copy (the tail
            // up to the next multiple of 16 bytes may not be readable there, so it goes through the staging buffer)
            const size_t whole = len & ~size_t(15);
            GTOK_CUDA(cudaMemcpyAsync(d_dst, src, whole, cudaMemcpyHostToDevice, stream));
            if (len > whole) {
                std::memcpy(h_pin, src + whole, len - whole);
                GTOK_CUDA(cudaMemcpyAsync(d_dst + whole, h_pin, 16, cudaMemcpyHostToDevice, stream));
            }
            return true;
        }
        if (pool && len >= 2 * kCopyPart) {
            const int parts = static_cast<int>((len + kCopyPart - 1) / kCopyPart);
            if (part_done_n < parts) { part_done.reset(new std::atomic<uint8_t>[parts]); part_done_n = parts; }
            for (int p = 0; p < parts; ++p) part_done[p].store(0, std::memory_order_relaxed);
            const std::function<void(int)> fn = [&](int p) {
                const size_t off = static_cast<size_t>(p) * kCopyPart;
                std::memcpy(h_pin + off, src + off, std::min(kCopyPart, len - off));
                part_done[p].store(1, std::memory_order_release);
            };
            pool->start(parts, &fn);
            int issued = 0;
            cudaError_t ce = cudaSuccess;
            while (issued < parts) {
                int upto = issued;
                while (upto < parts && part_done[upto].load(std::memory_order_acquire)) ++upto;
                if (upto > issued) {
                    const size_t off = static_cast<size_t>(issued) * kCopyPart;
                    const size_t end = std::min(static_cast<size_t>(upto) * kCopyPart, len);
                    const cudaError_t e1 = cudaMemcpyAsync(d_dst + off, h_pin + off, (end - off + 15) & ~size_t(15), cudaMemcpyHostToDevice, stream);
                    if (ce == cudaSuccess) ce = e1;
                    issued = upto;
                    continue;
                }
                const int p = pool->take();
                if (p >= 0) { fn(p); pool->done_one(); } else CopyPool::cpu_relax();
            }
            pool->finish();
            if (ce != cudaSuccess) { err = std::string("copy to the device: ") + cudaGetErrorString(ce); return false; }
        } else {
            std::memcpy(h_pin, src, len);
            GTOK_CUDA(cudaMemcpyAsync(d_dst, h_pin, (len + 15) & ~size_t(15), cudaMemcpyHostToDevice, stream));
        }
        return true;
    }

    // Host -> pinned -> device, for the text and the header.
    // With NFC the destination is the raw buffer; `normalised`: the text has been normalised on the host, the graph need not look.
    bool stage_input(Ctx* c, const uint8_t* bytes, uint32_t len, const uint32_t* doc_off, uint32_t n_docs, std::string& err,
                     bool normalised = false) {
        uint8_t* d_dst = nfc ? c->d_raw : c->d_text;
        if (len && !host_to_device(d_dst, c->h_text, bytes, len, c->stream, err)) return false;
        c->h_hdr[0] = len;
        c->h_hdr[1] = n_docs;
        c->h_hdr[2] = normalised ? 1u : 0u;
        c->h_hdr[3] = 0;
        size_t hdr_words = kHdrWords;
        if (doc_off) {
            std::memcpy(c->h_hdr + kHdrWords, doc_off, (static_cast<size_t>(n_docs) + 1) * 4);
            hdr_words += static_cast<size_t>(n_docs) + 1;
        }
        GTOK_CUDA(cudaMemcpyAsync(nfc ? c->d_rawhdr : c->d_hdr, c->h_hdr, hdr_words * 4, cudaMemcpyHostToDevice, c->stream));
        c->staged_len = len;
        c->staged_docs = n_docs;
        return true;
    }

    // Device -> pinned -> the caller's memory, then the stream is idle.  Large outputs part by part,
    // so that the copy out of pinned memory of one part overlaps with the DMA of the next ones.
    bool device_to_host(void* out, void* h_pin, const void* d_src, size_t bytes, cudaStream_t stream, cudaEvent_t* evs, std::string& err) {
        if (pool && bytes >= 2 * kCopyPart) {
            size_t part = kCopyPart;
            while ((bytes + part - 1) / part > static_cast<size_t>(kCopyEvents)) part *= 2;
            const int parts = static_cast<int>((bytes + part - 1) / part);
            for (int p = 0; p < parts; ++p) {
                if (!evs[p]) GTOK_CUDA(cudaEventCreateWithFlags(&evs[p], cudaEventDisableTiming));
                const size_t off = static_cast<size_t>(p) * part, nb = std::min(part, bytes - off);
                GTOK_CUDA(cudaMemcpyAsync(static_cast<char*>(h_pin) + off, static_cast<const char*>(d_src) + off, nb, cudaMemcpyDeviceToHost, stream));
                GTOK_CUDA(cudaEventRecord(evs[p], stream));
            }
            // pieces arrive in order; this thread watches the events and publishes how many are in,
            // every thread (this one too) copies arrived pieces out of pinned memory
            std::atomic<int> ready{0};
            std::atomic<int> failed{0};
            const std::function<void(int)> fn = [&](int p) {
                while (ready.load(std::memory_order_acquire) <= p && !failed.load(std::memory_order_relaxed)) CopyPool::cpu_relax();
                if (failed.load(std::memory_order_relaxed)) return;
                const size_t off = static_cast<size_t>(p) * part, nb = std::min(part, bytes - off);
                std::memcpy(static_cast<char*>(out) + off, static_cast<const char*>(h_pin) + off, nb);
            };
            pool->start(parts, &fn);
            int in = 0;
            cudaError_t ce = cudaSuccess;
            while (in < parts) {
                const cudaError_t q = cudaEventQuery(evs[in]);
                if (q == cudaSuccess) { ready.store(++in, std::memory_order_release); continue; }
                if (q != cudaErrorNotReady) { ce = q; failed.store(1); break; }
                CopyPool::cpu_relax();
            }
            for (int p; (p = pool->take()) >= 0;) { fn(p); pool->done_one(); }
            pool->finish();
            if (ce != cudaSuccess) { err = std::string("copy from the device: ") + cudaGetErrorString(ce); return false; }
            GTOK_CUDA(cudaStreamSynchronize(stream));
        } else {
            if (bytes) GTOK_CUDA(cudaMemcpyAsync(h_pin, d_src, bytes, cudaMemcpyDeviceToHost, stream));
            GTOK_CUDA(cudaStreamSynchronize(stream));
            if (bytes) std::memcpy(out, h_pin, bytes);
        }
        return true;
    }

    // Is this host pointer page-locked memory the device can reach (cudaHostAlloc / cudaHostRegister)?
    static bool is_pinned(const void* p) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
        return at.type == cudaMemoryTypeHost;
    }

    // ids (and, for a batch, the document offsets behind them) from the device to the caller's
    // memory: directly when that is page-locked, else through the pinned buffer.
    bool copy_out(Ctx* c, uint32_t* out, size_t words, uint32_t* out_doc_tok, size_t doc_words, std::string& err) {
        const size_t bytes = words * 4;
        if (words && bytes >= kCopyPart && is_pinned(out)) {
            // the caller's buffer is page-locked: the ids go there directly, no staging copy
            GTOK_CUDA(cudaMemcpyAsync(out, c->d_out, bytes, cudaMemcpyDeviceToHost, c->stream));
            if (doc_words) {
                if (!grow_host_out(c, doc_words + 2, err)) return false;
                GTOK_CUDA(cudaMemcpyAsync(c->h_out, c->d_doc_tok, doc_words * 4, cudaMemcpyDeviceToHost, c->stream));
            }
            GTOK_CUDA(cudaStreamSynchronize(c->stream));
            if (doc_words) std::memcpy(out_doc_tok, c->h_out, doc_words * 4);
            return true;
        }
        if (!grow_host_out(c, words + doc_words + 2, err)) return false;
        if (doc_words) GTOK_CUDA(cudaMemcpyAsync(c->h_out + words, c->d_doc_tok, doc_words * 4, cudaMemcpyDeviceToHost, c->stream));
        if (!device_to_host(out, c->h_out, c->d_out, bytes, c->stream, c->out_ev, err)) return false;
        if (doc_words) std::memcpy(out_doc_tok, c->h_out + words, doc_words * 4);
        return true;
    }

    static constexpr int64_t kNoCtx = INT64_MIN;

    // Stages the input and replays the graph.  With NFC two things can make the first replay
    // give up, and each is retried once: a stretch longer than a thread normalises (the text is
    // then normalised on the host and the kernel only copies it), and normalised text longer
    // than the text buffer (the context is rebuilt larger; NFC grows a text at most threefold).
    int64_t run(Ctx*& c, bool batch_mode, const uint8_t* bytes, uint32_t len, const uint32_t* doc_off, uint32_t n_docs,
                uint32_t cap_hint, std::string& err) {
        c = ctx_for(batch_mode, len, n_docs, cap_hint, err);
        if (!c) return kNoCtx;
        if (!stage_input(c, bytes, len, doc_off, n_docs, err)) return -1;
        int64_t total = replay(c, false, nullptr, err);
        if (total >= 0 || !nfc || !(last_err_bits & (kErrNfcLong | kErrNfcFull))) return total;
        if (last_err_bits & kErrNfcLong) {
            norm.clear();
            if (!batch_mode) {
                if (!nfc_normalize(bytes, len, norm)) norm.assign(reinterpret_cast<const char*>(bytes), len);
            } else {
                norm_off.assign(static_cast<size_t>(n_docs) + 1, 0);
                for (uint32_t i = 0; i < n_docs; ++i) {
                    const uint8_t* d = bytes + doc_off[i];
                    const uint32_t dl = doc_off[i + 1] - doc_off[i];
                    if (nfc_normalize(d, dl, norm_doc)) norm += norm_doc;
                    else norm.append(reinterpret_cast<const char*>(d), dl);
                    if (norm.size() > 0xFFFFFF00ull) { err = "normalised text exceeds 4 GiB"; return -3; }
                    norm_off[i + 1] = static_cast<uint32_t>(norm.size());
                }
            }
            if (norm.size() > 0xFFFFFF00ull) { err = "normalised text exceeds 4 GiB"; return -3; }
            if (norm.empty()) { c->h_status[0] = 0; c->h_status[2] = 0; return 0; }
            const uint32_t nl = static_cast<uint32_t>(norm.size());
            c = ctx_for(batch_mode, nl, n_docs, cap_hint, err);
            if (!c) return kNoCtx;
            if (!stage_input(c, reinterpret_cast<const uint8_t*>(norm.data()), nl, batch_mode ? norm_off.data() : nullptr, n_docs, err, true)) return -1;
            return replay(c, false, nullptr, err);
        }
        const uint64_t want = static_cast<uint64_t>(len) * 3 + 64;
        if (want > 0xFFFFFF00ull) { err = "normalised text may exceed 4 GiB"; return -3; }
        c = ctx_for(batch_mode, static_cast<uint32_t>(want), n_docs, cap_hint, err);
        if (!c) return kNoCtx;
        if (!stage_input(c, bytes, len, doc_off, n_docs, err)) return -1;
        return replay(c, false, nullptr, err);
    }

    // One replay; returns the total token count or -1.
    int64_t replay(Ctx* c, bool timed, float* ms, std::string& err) {
        c->h_status[0] = 0;
        c->h_status[1] = 0;
        c->h_status[2] = c->staged_len;
        last_err_bits = 0;
        if (c->staged_len == 0) { if (ms) *ms = 0.f; return 0; }
        auto fail = [&](cudaError_t e, const char* what) { err = std::string(what) + ": " + cudaGetErrorString(e); return int64_t(-1); };
        cudaError_t e;
        if (timed && (e = cudaEventRecord(c->ev[0], c->stream)) != cudaSuccess) return fail(e, "cudaEventRecord");
        if ((e = cudaGraphLaunch(c->exec, c->stream)) != cudaSuccess) return fail(e, "cudaGraphLaunch");
        if (timed && (e = cudaEventRecord(c->ev[1], c->stream)) != cudaSuccess) return fail(e, "cudaEventRecord");
        if ((e = cudaStreamSynchronize(c->stream)) != cudaSuccess) return fail(e, "cudaStreamSynchronize");
        if (timed && ms) cudaEventElapsedTime(ms, c->ev[0], c->ev[1]);
        uint32_t errs = reinterpret_cast<volatile uint32_t*>(c->h_status)[1];
        if (errs) {
            last_err_bits = errs;
            char buf[96];
            std::snprintf(buf, sizeof buf, "encode kernels reported error bits 0x%x", errs);
            err = buf;
            return (errs & kErrOutputFull) ? -2 : -1;
        }
        return reinterpret_cast<volatile uint32_t*>(c->h_status)[0];
    }
};

Engine::~Engine() = default;

Engine* Engine::create(const std::string& path, std::string& err) {
    std::unique_ptr<Engine> e(new Engine());
    if (!load_tokenizer_json(path, e->hv_, err)) return nullptr;
    e->impl_.reset(new Impl());
    Impl& im = *e->impl_;
    if (!build_host_tables(e->hv_, im.ht, err)) return nullptr;
    int n_dev = 0;
    cudaError_t ce = cudaGetDeviceCount(&n_dev);
    if (ce != cudaSuccess || n_dev == 0) {
        err = std::string("no CUDA device: ") + (ce != cudaSuccess ? cudaGetErrorString(ce) : "device count is 0") +
              " (this library has no CPU path)";
        return nullptr;
    }
    int dev = 0;
    if (const char* env = std::getenv("GTOK_DEVICE")) dev = std::atoi(env);
    else cudaGetDevice(&dev);
    if (cudaSetDevice(dev) != cudaSuccess) { err = "cudaSetDevice failed"; return nullptr; }
    im.device = dev;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { err = "cudaGetDeviceProperties failed"; return nullptr; }
    im.sm_count = prop.multiProcessorCount;
    if (prop.major < 10) {
        err = "this build targets sm_100a (B200); found compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor);
        return nullptr;
    }
    if (configure_kernels() != cudaSuccess) { err = std::string("kernel configuration failed: ") + cudaGetErrorString(cudaGetLastError()); return nullptr; }
    im.pretok_per_sm = pretok_blocks_per_sm();
    im.words_per_sm = words_blocks_per_sm();
    im.miss_per_sm = miss_blocks_per_sm();
    im.asm_per_sm = assemble_blocks_per_sm();
    im.nfc_per_sm = nfc_blocks_per_sm();
    im.nfc = e->hv_.nfc;
    if (const char* env = std::getenv("GTOK_TINY")) im.tiny = std::atoi(env) != 0;
    if (im.tiny && configure_tiny_kernel() != cudaSuccess) { err = std::string("kernel configuration failed: ") + cudaGetErrorString(cudaGetLastError()); return nullptr; }
    if (!im.upload_tables(err)) return nullptr;
    im.reserve_l2();
    {
        // GTOK_COPY_THREADS = host threads that share one call's staging copies (1 = the caller alone)
        int want = 4;
        if (const char* env = std::getenv("GTOK_COPY_THREADS")) want = std::atoi(env);
        int hw = static_cast<int>(std::thread::hardware_concurrency());
        if (hw > 0) {
            // at most half the cores; with one process per GPU (torchrun exports LOCAL_WORLD_SIZE) this engine's share of them
            int share = hw / 2;
            if (const char* lws = std::getenv("LOCAL_WORLD_SIZE")) { const int k = std::atoi(lws); if (k > 1) share = hw / k; }
            want = std::min(want, std::max(1, share));
        }
        want = std::min(want, 16);
        // Workers poll for 1.5 ms after a job, so that the copy-out of a call finds them awake after its
        // copy-in; with several ranks on one host (torchrun exports LOCAL_WORLD_SIZE) that polling would
        // take cores from the other ranks' copies, so they go to sleep almost at once.
        int spin_us = 1500;
        if (const char* lws = std::getenv("LOCAL_WORLD_SIZE")) { if (std::atoi(lws) > 1) spin_us = 40; }
        if (want > 1) im.pool.reset(new CopyPool(want - 1, spin_us));
    }
    return e.release();
}

void Engine::table_bytes(uint64_t* merge, uint64_t* word, uint64_t* other) const {
    const HostTables& ht = impl_->ht;
    *merge = ht.merge.size() * sizeof(MergeSlot);
    *word = ht.word.size() * sizeof(WordSlot);
    *other = ht.longtab.size() * sizeof(LongSlot) + ht.long_blob.size() + 1024 + GTOK_UC_STAGE1_LEN * 2 + GTOK_UC_STAGE2_LEN * 4;
}

int64_t Engine::encode(const uint8_t* text, uint32_t len, uint32_t cap_bytes, uint32_t* out, uint32_t max_out, bool out_on_device) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    if (len == 0) return 0;
    if (!out_on_device && len <= kTinyMaxBytes && im.tiny && !im.nfc) {
        Ctx* tc = im.ctx_for(false, len, 1, cap_bytes, last_error_);
        if (!tc) return -1;
        if (tc->tiny_exec) {
            const int64_t r = im.run_tiny(tc, text, len, out, max_out, last_error_);
            if (r != Impl::kNoCtx) return r;
        }
    }
    Ctx* c = nullptr;
    int64_t total = im.run(c, false, text, len, nullptr, 1, cap_bytes, last_error_);
    if (total == Impl::kNoCtx) return -1;
    if (total < 0) return total;
    if (im.nfc && c->h_status[2] > cap_bytes) { last_error_ = "normalised text is longer than the handle's byte capacity"; return -3; }
    if (static_cast<uint64_t>(total) > max_out) { last_error_ = "more token ids than the output buffer holds"; return -2; }
    if (total == 0) return 0;
    if (out_on_device) {
        cudaError_t e = cudaMemcpyAsync(out, c->d_out, static_cast<size_t>(total) * 4, cudaMemcpyDeviceToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { last_error_ = std::string("token copy: ") + cudaGetErrorString(e); return -1; }
    } else if (!im.copy_out(c, out, static_cast<size_t>(total), nullptr, 0, last_error_)) return -1;
    return total;
}

int64_t Engine::encode_batch(const uint8_t* bytes, const uint32_t* doc_off, uint32_t n_docs, uint32_t cap_bytes,
                             uint32_t* out_tokens, uint32_t out_cap, uint32_t* out_doc_tok, bool out_on_device) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    const uint32_t len = doc_off[n_docs];
    if (len == 0) {
        if (out_on_device) { if (cudaMemset(out_doc_tok, 0, (static_cast<size_t>(n_docs) + 1) * 4) != cudaSuccess) return -1; }
        else for (uint32_t d = 0; d <= n_docs; ++d) out_doc_tok[d] = 0;
        return 0;
    }
    Ctx* c = nullptr;
    int64_t total = im.run(c, true, bytes, len, doc_off, n_docs, cap_bytes, last_error_);
    if (total == Impl::kNoCtx) return -4;
    if (total < 0) return total;
    if (im.nfc && c->h_status[2] > cap_bytes) { last_error_ = "normalised text is longer than the handle's byte capacity"; return -3; }
    if (static_cast<uint64_t>(total) > out_cap) { last_error_ = "more token ids than the output buffer holds"; return -2; }
    if (out_on_device) {
        cudaError_t e = cudaSuccess;
        if (total) e = cudaMemcpyAsync(out_tokens, c->d_out, static_cast<size_t>(total) * 4, cudaMemcpyDeviceToDevice, c->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(out_doc_tok, c->d_doc_tok, (static_cast<size_t>(n_docs) + 1) * 4, cudaMemcpyDeviceToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { last_error_ = std::string("token copy: ") + cudaGetErrorString(e); return -1; }
        return total;
    }
    if (!im.copy_out(c, out_tokens, static_cast<size_t>(total), out_doc_tok, static_cast<size_t>(n_docs) + 1, last_error_)) return -1;
    return total;
}

int Engine::stage(const uint8_t* bytes, uint32_t len, const uint32_t* doc_off, uint32_t n_docs, uint32_t cap_bytes) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    const bool batch_mode = doc_off != nullptr;
    Ctx* c = im.ctx_for(batch_mode, len, batch_mode ? n_docs : 1, cap_bytes, last_error_);
    if (!c) return -1;
    if (!im.stage_input(c, bytes, len, doc_off, batch_mode ? n_docs : 1, last_error_)) return -1;
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) { last_error_ = "stage: stream synchronize failed"; return -1; }
    im.staged = c;
    return 0;
}

int64_t Engine::replay_staged(float* ms_out) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    if (!im.staged) { last_error_ = "nothing staged"; return -1; }
    return im.replay(im.staged, true, ms_out, last_error_);
}

int64_t Engine::profile_staged(float* ms_out) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c) { last_error_ = "nothing staged"; return -1; }
    c->h_status[0] = 0;
    c->h_status[1] = 0;
    for (int i = 0; i < 6; ++i) ms_out[i] = 0.f;
    if (c->staged_len == 0) return 0;
    cudaEventRecord(c->ev[0], c->stream);
    cudaMemsetAsync(c->d_ctrl, 0, c->ctrl_bytes, c->stream);
    cudaEventRecord(c->ev[6], c->stream);
    im.launch_front(c);
    cudaEventRecord(c->ev[1], c->stream);
    launch_pretok(c->args, c->pretok_blocks, c->stream);
    cudaEventRecord(c->ev[2], c->stream);
    launch_words(c->args, c->words_blocks, c->stream);
    cudaEventRecord(c->ev[3], c->stream);
    launch_miss(c->args, c->miss_blocks, c->stream);
    cudaEventRecord(c->ev[4], c->stream);
    launch_assemble(c->args, c->asm_blocks, c->stream);
    cudaEventRecord(c->ev[5], c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { last_error_ = std::string("profile: ") + cudaGetErrorString(e); return -1; }
    for (int i = 0; i < 4; ++i) cudaEventElapsedTime(&ms_out[i], c->ev[i + 1], c->ev[i + 2]);
    cudaEventElapsedTime(&ms_out[4], c->ev[0], c->ev[5]);
    cudaEventElapsedTime(&ms_out[5], c->ev[6], c->ev[1]);
    if (reinterpret_cast<volatile uint32_t*>(c->h_status)[1]) { last_error_ = "encode kernels reported an error"; return -1; }
    return reinterpret_cast<volatile uint32_t*>(c->h_status)[0];
}

int64_t Engine::read_boundaries(uint32_t* out_words, uint32_t max_words) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c) { last_error_ = "nothing staged"; return -1; }
    const uint32_t text_bytes = im.nfc ? reinterpret_cast<volatile uint32_t*>(c->h_status)[2] : c->staged_len;
    uint32_t words = (text_bytes + 31) / 32;
    if (words > max_words) return -2;
    if (words && cudaMemcpy(out_words, c->d_bmask, static_cast<size_t>(words) * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return words;
}

int Engine::read_phase_clocks(unsigned long long* out32, bool reset) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c || !c->d_phase) return -1;
    if (cudaMemcpy(out32, c->d_phase, 32 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (reset) cudaMemset(c->d_phase, 0, 32 * sizeof(unsigned long long));
    return 0;
}

int Engine::read_work_stats(uint64_t* out6) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c) { last_error_ = "nothing staged"; return -1; }
    for (int i = 0; i < 6; ++i) out6[i] = 0;
    uint32_t ctl[16];
    if (cudaMemcpy(ctl, c->d_ctrl, sizeof ctl, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    const uint32_t text_bytes = im.nfc ? reinterpret_cast<volatile uint32_t*>(c->h_status)[2] : c->staged_len;
    const uint32_t n_tiles = (text_bytes + kTile - 1) / kTile;
    std::vector<uint32_t> bits(static_cast<size_t>(n_tiles) * kTileWords);
    if (!bits.empty() && cudaMemcpy(bits.data(), c->d_bmask, bits.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    for (uint32_t w : bits) out6[0] += static_cast<uint64_t>(__builtin_popcount(w));
    auto add_list = [&](const unsigned long long* d_list, long long dir, uint32_t count, uint64_t& n, uint64_t& bytes) -> bool {
        if (!count) return true;
        std::vector<unsigned long long> v(count);
        const unsigned long long* src = dir > 0 ? d_list : d_list - (count - 1);
        if (cudaMemcpy(v.data(), src, static_cast<size_t>(count) * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
        n += count;
        for (unsigned long long e : v) bytes += e >> 32;
        return true;
    };
    const EncodeArgs& a = c->args;
    if (!add_list(a.gmiss, 1, ctl[CTL_NMISS], out6[1], out6[2]) || !add_list(a.gmed, 1, ctl[CTL_NMED], out6[1], out6[2]) ||
        !add_list(a.gmed1, 1, ctl[CTL_NMED1], out6[1], out6[2]) || !add_list(a.gmed + (a.gmed_cap - 1), -1, ctl[CTL_NMED2], out6[1], out6[2]))
        return -1;
    const uint32_t n_long = ctl[CTL_NLONG];
    if (n_long) {
        std::vector<uint32_t> g(n_long), cnt(n_long);
        if (cudaMemcpy(g.data(), a.glong_g, static_cast<size_t>(n_long) * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
            cudaMemcpy(cnt.data(), a.glong_cnt, static_cast<size_t>(n_long) * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
            return -1;
        out6[3] = n_long;
        // a long pre-token ends at the next boundary bit
        for (uint32_t i = 0; i < n_long; ++i) {
            uint32_t p = g[i] + 1;
            while (p < text_bytes && !((bits[p >> 5] >> (p & 31)) & 1u)) ++p;
            out6[4] += p - g[i];
            out6[5] += cnt[i];
        }
    }
    // ids written by the miss kernel = all ids - one per pre-token the earlier kernels settled
    const uint64_t total = reinterpret_cast<volatile uint32_t*>(c->h_status)[0];
    const uint64_t settled = out6[0] - out6[1] - out6[3];
    out6[5] = total > settled ? total - settled : 0;
    return 0;
}

int Engine::read_timeline(unsigned long long* out, uint32_t max_words) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c || !c->d_phase) return -1;
    const uint32_t words = std::min<uint32_t>(max_words, kTlWords);
    if (cudaMemcpy(out, c->d_phase + kPhaseWords, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    cudaMemset(c->d_phase + kPhaseWords, 0, kTlWords * sizeof(unsigned long long));
    return static_cast<int>(words);
}

// ids -> bytes on the device (the reference's TokenizerCtx::decode, src/tokenizer.cu:5499-5573).
int64_t Engine::decode(const uint32_t* ids, uint32_t n, uint8_t* out, uint64_t max_out, uint64_t* need, float* kernel_ms) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    if (need) *need = 0;
    if (kernel_ms) *kernel_ms = 0.f;
    if (n == 0) return 0;
    if (!im.upload_decode_tables(hv_, last_error_)) return -1;
    const uint64_t most = static_cast<uint64_t>(n) * std::max<uint32_t>(im.max_tok_len, 1);
    if (most > 0xFFFFFFF0ull && max_out > 0xFFFFFFF0ull) max_out = 0xFFFFFFF0ull;    // byte offsets are 32-bit on the device
    // The device buffer starts at 16 bytes per id (spellings average 4-5) and grows to the measured
    // byte count when that was not enough, rather than to the caller's bound or the longest spelling
    // times the count.
    const uint64_t bound = std::max<uint64_t>(std::min<uint64_t>(most, max_out), 1024);
    uint64_t want = std::min<uint64_t>(bound, 16ull * n + 4096);
    DecCtx* c = nullptr;
    uint32_t total = 0, bits = 0;
    for (int attempt = 0; attempt < 2; ++attempt) {
        if (!im.dec || im.dec->cap_ids < n || im.dec->cap_bytes < want) {
            uint32_t cap_ids = 4096;
            while (cap_ids < n && cap_ids < 0x80000000u) cap_ids <<= 1;
            if (cap_ids < n) cap_ids = n;
            size_t cap_bytes = 16384;
            while (cap_bytes < want) cap_bytes <<= 1;
            if (im.dec) { cap_ids = std::max(cap_ids, im.dec->cap_ids); cap_bytes = std::max(cap_bytes, im.dec->cap_bytes); }
            im.dec.reset();
            if (!im.build_dec(cap_ids, cap_bytes, hv_.vocab_size, last_error_)) { im.dec.reset(); return -1; }
        }
        c = im.dec.get();
        c->h_in[0] = n;
        c->h_in[1] = c->h_in[2] = c->h_in[3] = 0;
        cudaError_t e = cudaMemcpyAsync(c->d_in, c->h_in, 16, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess && !im.host_to_device(reinterpret_cast<uint8_t*>(c->d_in + 4), reinterpret_cast<uint8_t*>(c->h_in + 4),
                                                   reinterpret_cast<const uint8_t*>(ids), static_cast<size_t>(n) * 4, c->stream, last_error_))
            return -1;
        if (e == cudaSuccess) e = cudaEventRecord(c->ev[0], c->stream);
        if (e == cudaSuccess) e = cudaGraphLaunch(c->exec, c->stream);
        if (e == cudaSuccess) e = cudaEventRecord(c->ev[1], c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { last_error_ = std::string("decode: ") + cudaGetErrorString(e); return -1; }
        if (kernel_ms) cudaEventElapsedTime(kernel_ms, c->ev[0], c->ev[1]);
        total = c->h_status[0];
        bits = c->h_status[1];
        // the count is exact even when the buffer was too small: once more with room for it
        if ((bits & kErrOutputFull) && !(bits & (kErrBadId | kErrWaitExpired)) && total > c->cap_bytes && total <= bound) { want = total; continue; }
        break;
    }
    cudaError_t e = cudaSuccess;
    if (bits & kErrBadId) { last_error_ = "decode: an id is outside the vocabulary"; return -1; }
    if (bits & kErrWaitExpired) { last_error_ = "decode: a wait on an earlier tile gave up"; return -1; }
    if (total == 0xFFFFFFFFu) { last_error_ = "decode: the ids spell 4 GiB or more, beyond what one call decodes"; return -1; }
    if (need) *need = total;
    if ((bits & kErrOutputFull) || total > max_out) { last_error_ = "decode: more bytes than the output buffer holds"; return -2; }
    if (bits) { last_error_ = "decode: internal error"; return -1; }
    if (total == 0) return 0;
    if (im.is_pinned(out)) {
        e = cudaMemcpyAsync(out, c->d_out, total, cudaMemcpyDeviceToHost, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    } else if (!im.device_to_host(out, c->h_out, c->d_out, total, c->stream, c->out_ev, last_error_)) return -1;
    if (e != cudaSuccess) { last_error_ = std::string("decode copy: ") + cudaGetErrorString(e); return -1; }
    return total;
}

const DeviceTables* Engine::device_tables() const { return &impl_->dt; }
int Engine::device_index() const { return impl_->device; }

int64_t Engine::read_staged(uint32_t* out, uint32_t max_out, uint32_t* out_doc_tok) {
    Impl& im = *impl_;
    cudaSetDevice(im.device);
    Ctx* c = im.staged;
    if (!c) { last_error_ = "nothing staged"; return -1; }
    uint32_t total = reinterpret_cast<volatile uint32_t*>(c->h_status)[0];
    if (total > max_out) return -2;
    if (total && cudaMemcpy(out, c->d_out, static_cast<size_t>(total) * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (out_doc_tok && c->batch &&
        cudaMemcpy(out_doc_tok, c->d_doc_tok, (static_cast<size_t>(c->staged_docs) + 1) * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    return total;
}

}  // namespace gtok
