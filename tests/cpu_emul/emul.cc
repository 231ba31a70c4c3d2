// Serial CPU emulation of the encode kernels' thread blocks, for tests only.
// The tile programs in graphtok_b200/csrc/encode_core.h are templates over a
// "block" object; here that object runs the 256 logical threads of a block one
// after the other (forwards or backwards, so that a dependence on thread order
// shows up as a difference between the two), and the tiles in order.  This lets
// the CPU test suite check the kernels' logic against the oracle without a GPU.
// It is not part of the shipped library and not a fallback: libgtok has no CPU path.
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../graphtok_b200/csrc/decode_core.h"
#include "../../graphtok_b200/csrc/encode_core.h"
#include "../../graphtok_b200/csrc/nfc_core.h"
#include "../../graphtok_b200/csrc/nfc_host.h"
#include "../../graphtok_b200/csrc/shard_plan.h"
#include "../../graphtok_b200/csrc/tables_build.h"
#include "../../graphtok_b200/csrc/unicode_class_table.h"
#include "../../graphtok_b200/csrc/unicode_wide_table.h"
#include "../../graphtok_b200/csrc/vocab_host.h"

namespace {

struct CpuBlk {
    bool reverse = false;
    // Per-thread values that live from one par() to the next: one copy per logical thread.
    template <class T>
    struct Local {
        T v[gtok::kThreads];
        T& at(int tid) { return v[tid]; }
    };
    template <class F> void par(F f) {
        if (!reverse) for (int t = 0; t < gtok::kThreads; ++t) f(t);
        else for (int t = gtok::kThreads - 1; t >= 0; --t) f(t);
    }
    void excl_scan(uint32_t* arr, uint32_t* total) {
        uint32_t acc = 0;
        for (int i = 0; i < gtok::kThreads; ++i) { uint32_t v = arr[i]; arr[i] = acc; acc += v; }
        *total = acc;
    }
    void excl_scan_and_sum(uint32_t* arr, uint32_t* total, const uint32_t* other, uint32_t* other_total) {
        uint32_t o = 0;
        for (int i = 0; i < gtok::kThreads; ++i) o += other[i];
        excl_scan(arr, total);
        *other_total = o;
    }
    uint32_t lookback(unsigned long long* st, int tile, uint32_t total, uint32_t*) {
        unsigned long long base = 0;         // saturating, like the kernels' look-back
        for (int j = tile - 1; j >= 0; --j) {
            base += static_cast<uint32_t>(st[j]);
            if ((st[j] >> 62) == 2) break;
        }
        if (base > 0xFFFFFFFFull) base = 0xFFFFFFFFull;
        st[tile] = gtok::kStFinal | (base + total > 0xFFFFFFFFull ? 0xFFFFFFFFull : base + total);
        return static_cast<uint32_t>(base);
    }
    uint32_t reduce_min(uint32_t* arr) {
        uint32_t m = 0xFFFFFFFFu;
        for (int i = 0; i < gtok::kThreads; ++i) if (arr[i] < m) m = arr[i];
        return m;
    }
};

struct Emul {
    gtok::HostVocab hv;
    gtok::HostTables ht;
    gtok::DeviceTables tb;
    std::vector<uint16_t> s1;
    std::vector<uint32_t> s2;
};

}  // namespace

static uint32_t g_last_ctl[16];

extern "C" {

void* gtok_emul_create(const char* path, char* err, uint32_t err_cap) {
    Emul* e = new Emul();
    std::string msg;
    if (!gtok::load_tokenizer_json(path, e->hv, msg) || !gtok::build_host_tables(e->hv, e->ht, msg)) {
        if (err && err_cap) { std::strncpy(err, msg.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
        delete e;
        return nullptr;
    }
    e->s1.assign(gtok_uc_stage1_init, gtok_uc_stage1_init + GTOK_UC_STAGE1_LEN);
    e->s2.assign(gtok_uc_stage2_init, gtok_uc_stage2_init + GTOK_UC_STAGE2_LEN);
    if (e->ht.family == 3) {
        e->s1.assign(gtok_uw_stage1_init, gtok_uw_stage1_init + GTOK_UW_STAGE1_LEN);
        e->s2.assign(gtok_uw_stage2_init, gtok_uw_stage2_init + GTOK_UW_STAGE2_LEN);
    }
    if (e->ht.family == 4) { e->s1 = e->ht.sp_stage1; e->s2 = e->ht.sp_stage2; }
    gtok::DeviceTables& tb = e->tb;
    const gtok::HostTables& ht = e->ht;
    tb.merge = ht.merge.data();
    tb.word = ht.word.data();
    tb.longtab = ht.longtab.data();
    tb.long_blob = ht.long_blob.data();
    tb.byte_to_id = ht.byte_to_id.data();
    tb.uc_stage1 = e->s1.data(); tb.uc_stage2 = e->s2.data();
    tb.trie_root = ht.trie_root.data(); tb.trie_first = ht.trie_first.data(); tb.trie_count = ht.trie_count.data();
    tb.trie_terminal = ht.trie_terminal.data(); tb.trie_edges = ht.trie_edges.data();
    tb.trie_skip = ht.trie_skip.data(); tb.trie_blob = ht.trie_blob.data();
    tb.littab = ht.littab.data();
    static_assert(GTOK_UC_STAGE2_LEN == gtok::kUcStage2Words && GTOK_UC_STAGE1_LEN >= gtok::kUcStage1Bmp, "class table sizes");
    gtok::fill_table_scalars(ht, tb);
    return e;
}

void gtok_emul_destroy(void* h) { delete static_cast<Emul*>(h); }

// force_non_monotone: bit 0 treats the vocabulary as non-monotone (exercises the one-merge-per-round path),
// bit 1 matches added-token literals by the trie walk (the path of vocabularies with too many literal lengths to hash)
// Returns the token count, or -(error bits) when the kernels flagged an error.
int64_t gtok_emul_encode(void* h, const uint8_t* text, uint32_t n, const uint32_t* doc_off, uint32_t n_docs,
                         uint32_t* out, uint32_t cap, uint32_t* out_doc_tok, uint32_t* bmask_out, int reverse,
                         int force_non_monotone) {
    Emul* e = static_cast<Emul*>(h);
    using namespace gtok;
    const uint32_t n_tiles = (n + kTile - 1) / kTile;
    if (n == 0) { if (out_doc_tok) for (uint32_t d = 0; d <= n_docs; ++d) out_doc_tok[d] = 0; return 0; }
    std::vector<uint8_t> buf(static_cast<size_t>(n_tiles) * kTile + kTile + kWin + 64, 0xAA);   // junk past n
    std::memcpy(buf.data(), text, n);
    uint32_t meta[2] = {n, n_docs};
    std::vector<uint32_t> docmask, bmask(n_tiles * kTileWords + 8, 0xDEADBEEF), amask(n_tiles * kTileWords + 8, 0xDEADBEEF), tile_nb(n_tiles + 1, 0);
    std::vector<unsigned long long> st1(n_tiles + 1, 0), st2(n_tiles + 1, 0);
    uint32_t ctl[16] = {0}, status[4] = {0, 0, 0, 0};
    std::vector<uint32_t> gstage(static_cast<size_t>(n_tiles) * kTile + 64), grk(gstage.size()), gnw(gstage.size());
    EncodeArgs a;
    std::memset(&a, 0, sizeof a);
    a.text = buf.data(); a.meta = meta;
    if (doc_off) {
        docmask.assign(n_tiles * kTileWords + 8, 0);
        for (uint32_t d = 0; d <= n_docs; ++d) if (doc_off[d] < n) docmask[doc_off[d] >> 5] |= 1u << (doc_off[d] & 31);
        a.doc_off = doc_off; a.docmask = docmask.data(); a.out_doc_tok = out_doc_tok;
    }
    std::vector<uint32_t> tile_tok(n_tiles + 1, 0);
    a.bmask = bmask.data(); a.amask = amask.data(); a.tile_nb = tile_nb.data(); a.tile_tok = tile_tok.data();
    a.sum_tiles = reverse ? 0u : static_cast<uint32_t>(kSumTiles);      // the reversed runs also take the look-back path of the assembly
    a.st1 = st1.data(); a.st2 = st2.data(); a.ctl = ctl;
    a.gstage = gstage.data(); a.gwork_rk = grk.data(); a.gwork_nw = gnw.data();
    std::vector<uint32_t> stage(gstage.size(), 0xABABABAB), ovf(static_cast<size_t>(n_tiles + 1) * kTokExtra, 0xABABABAB);
    std::vector<unsigned long long> gmiss(gstage.size() / 2 + 64), gmed(gstage.size() / 16 + 64), gmed1(gstage.size() / 32 + 64);
    std::vector<uint32_t> glong(static_cast<size_t>(n_tiles + 1) * kLongPerTile * 3, 0xABABABAB);
    a.stage = stage.data(); a.ovf = ovf.data(); a.gmiss = gmiss.data(); a.gmed = gmed.data(); a.gmed_cap = static_cast<uint32_t>(gmed.size()); a.gmed1 = gmed1.data();
    a.glong_g = glong.data(); a.glong_len = glong.data() + static_cast<size_t>(n_tiles + 1) * kLongPerTile;
    a.glong_cnt = glong.data() + static_cast<size_t>(n_tiles + 1) * kLongPerTile * 2;
    a.out_tokens = out; a.out_cap = cap; a.status = status;
    a.tb = e->tb;
    if (force_non_monotone & 1) a.tb.monotone = 0;
    if (force_non_monotone & 2) a.tb.lit_n_lens = 0;            // added-token literals by the trie walk instead of the hashed table
    CpuBlk blk;
    blk.reverse = reverse != 0;
    {
        PretokSmem* sm = new PretokSmem();
        for (uint32_t t = 0; t < (n + kPTile - 1) / kPTile; ++t) {
            std::memset(sm, 0xCD, sizeof *sm);
            if (a.tb.uc_wide) { pretok_block_init<true>(blk, a, *sm); pretok_tile<true>(blk, a, *sm, static_cast<int>(t)); }
            else { pretok_block_init<false>(blk, a, *sm); pretok_tile<false>(blk, a, *sm, static_cast<int>(t)); }
        }
        delete sm;
    }
    if (bmask_out) std::memcpy(bmask_out, bmask.data(), static_cast<size_t>(n_tiles) * kTileWords * 4);
    {
        WordsSmem* sm = new WordsSmem();
        // tiles of this kernel are independent: run them last to first to show it
        for (uint32_t t = n_tiles; t-- > 0;) { std::memset(sm, 0xCD, sizeof *sm); words_tile(blk, a, *sm, static_cast<int>(t)); }
        delete sm;
    }
    {
        MissSmem* sm = new MissSmem();
        std::memset(sm, 0xCD, sizeof *sm);
        for (int i = 0; i < 256; ++i) sm->b2i[i] = a.tb.byte_to_id[i];
        const uint32_t n_miss = ctl[CTL_NMISS], n_med = ctl[CTL_NMED], n_med1 = ctl[CTL_NMED1], n_med2 = ctl[CTL_NMED2], n_long = ctl[CTL_NLONG];
        for (uint32_t first = 0; first < n_med; first += kMedBatchA) miss_batch(blk, a, *sm, a.gmed, 1, first, n_med, kMedBatchA, kMedWordMax, kMedBatchA);
        for (uint32_t first = 0; first < n_med1; first += kMedBatchA1) miss_batch(blk, a, *sm, a.gmed1, 1, first, n_med1, kMedBatchA1, kMedSplit1, kMedBatchA1);
        const uint32_t take_b = a.tb.ignore_merges ? kMedTakeB : kMedBatchB;
        for (uint32_t first = 0; first < n_med2; first += take_b) {
            if (take_b > kMedBatchB) miss_batch_sharing(blk, a, *sm, a.gmed + (a.gmed_cap - 1), -1, first, n_med2, kMedBatchB, kMedSplit, take_b);
            else miss_batch(blk, a, *sm, a.gmed + (a.gmed_cap - 1), -1, first, n_med2, kMedBatchB, kMedSplit, take_b);
        }
        if (take_b > kMedBatchB)
            for (uint32_t first = 0; first < n_med2; first += take_b)
                for (uint32_t c = 0; c < kSurplusChunks; ++c) miss_surplus(blk, a, *sm, a.gmed + (a.gmed_cap - 1), -1, first, c);
        for (uint32_t first = 0; first < n_miss; first += kMissBatch) miss_batch(blk, a, *sm, a.gmiss, 1, first, n_miss, kMissBatch, kShortWordMax, kMissBatch);
        for (uint32_t li = 0; li < n_long; ++li) long_word(blk, a, *sm, li);
        delete sm;
    }
    {
        AsmSmem* sm = new AsmSmem();
        for (uint32_t t = 0; t < n_tiles; ++t) { std::memset(sm, 0xCD, sizeof *sm); assemble_tile(blk, a, *sm, static_cast<int>(t)); }
        delete sm;
    }
    std::memcpy(g_last_ctl, ctl, sizeof ctl);
    if (ctl[2]) return -static_cast<int64_t>(ctl[2]);
    return status[0];
}

// Control words of the last gtok_emul_encode (list sizes, error bits), for inspection.
const uint32_t* gtok_emul_last_ctl() { return g_last_ctl; }

// The library's host-side NFC (csrc/nfc_host.cc), reachable without a GPU handle.
int64_t gtok_emul_nfc(const uint8_t* text, uint64_t len, uint8_t* out, uint64_t cap) {
    std::string o;
    if (!gtok::nfc_normalize(text, len, o)) { if (len > cap) return -1; std::memcpy(out, text, len); return static_cast<int64_t>(len); }
    if (o.size() > cap) return -1;
    std::memcpy(out, o.data(), o.size());
    return static_cast<int64_t>(o.size());
}

// The device normaliser (csrc/nfc_core.h) run tile by tile on the CPU.  Returns the
// normalised length, or -(error bits).  `out` must hold `cap` bytes.
int64_t gtok_emul_nfc_device(const uint8_t* text, uint32_t n, const uint32_t* doc_off, uint32_t n_docs, uint8_t* out, uint32_t cap,
                             uint32_t* out_doc_off, int reverse, int already_normalised) {
    using namespace gtok;
    static NfcWords words;
    if (words.attn_bits.empty()) nfc_table_words(words);
    if (n == 0) { if (out_doc_off) for (uint32_t d = 0; d <= n_docs; ++d) out_doc_off[d] = 0; return 0; }
    const uint32_t n_tiles = (n + kTile - 1) / kTile;
    std::vector<uint8_t> raw(static_cast<size_t>(n_tiles) * kTile + kTile + kWin + 64, 0xCC);   // junk past n
    std::memcpy(raw.data(), text, n);
    std::vector<uint8_t> norm(static_cast<size_t>(cap) + 64, 0xEE);
    uint32_t raw_meta[4] = {n, n_docs, already_normalised ? 1u : 0u, 0}, meta[4] = {0, 0, 0, 0}, ctl[16] = {0}, status[4] = {0, 0, 0, 0};
    std::vector<uint32_t> docmask;
    std::vector<unsigned long long> st0(n_tiles + 1, 0);
    EncodeArgs a;
    std::memset(&a, 0, sizeof a);
    a.raw = raw.data(); a.raw_meta = raw_meta; a.norm_text = norm.data(); a.text = norm.data(); a.norm_meta = meta; a.meta = meta;
    a.st0 = st0.data(); a.ctl = ctl; a.status = status; a.text_cap = cap;
    if (doc_off) {
        docmask.assign(n_tiles * kTileWords + 8, 0);
        for (uint32_t d = 0; d <= n_docs; ++d) if (doc_off[d] < n) docmask[doc_off[d] >> 5] |= 1u << (doc_off[d] & 31);
        a.raw_doc_off = doc_off; a.raw_docmask = docmask.data(); a.norm_doc_off = out_doc_off;
    }
    a.tb.nfc_attn_bits = words.attn_bits.data();
    a.tb.nfc_attn_sup = words.attn_sup.data(); a.tb.nfc_attn_sup_n = static_cast<uint32_t>(words.attn_sup.size() / 2);
    a.tb.nfc_ccc = words.ccc.data(); a.tb.nfc_ccc_n = static_cast<uint32_t>(words.ccc.size() / 2);
    a.tb.nfc_decomp = words.decomp.data(); a.tb.nfc_decomp_n = static_cast<uint32_t>(words.decomp.size() / 6);
    a.tb.nfc_comp = words.comp.data(); a.tb.nfc_comp_n = static_cast<uint32_t>(words.comp.size() / 3);
    for (int i = 0; i < 8; ++i) a.tb.nfc_lead_quiet[i] = words.lead_quiet[i];
    a.tb.nfc_cp_hash = words.cp_hash.data(); a.tb.nfc_cp_hash_mask = static_cast<uint32_t>(words.cp_hash.size() / 2 - 1);
    a.tb.nfc_comp_hash = words.comp_hash.data(); a.tb.nfc_comp_hash_mask = static_cast<uint32_t>(words.comp_hash.size() / 4 - 1);
    CpuBlk blk;
    blk.reverse = reverse != 0;
    NfcSmem* sm = new NfcSmem();
    for (uint32_t t = 0; t < n_tiles; ++t) { std::memset(sm, 0xCD, sizeof *sm); nfc_tile(blk, a, *sm, static_cast<int>(t)); }
    delete sm;
    if (ctl[CTL_ERR]) return -static_cast<int64_t>(ctl[CTL_ERR]);
    std::memcpy(out, norm.data(), meta[0]);
    return meta[0];
}

// The shard planner of libgtok (gtok_x_plan_chunks), reachable without a GPU handle.
// The decode tile program (decode_core.h) on one serial "block", tiles in order.  Returns the byte
// count (whatever `cap` is); *err_bits receives the error bits the kernel would report.
int64_t gtok_emul_decode(void* h, const uint32_t* ids, uint32_t n, uint8_t* out, uint32_t cap, int reverse, uint32_t* err_bits) {
    Emul* e = static_cast<Emul*>(h);
    const gtok::HostVocab& hv = e->hv;
    std::vector<uint32_t> off(static_cast<size_t>(hv.vocab_size) + 1, 0);
    std::vector<uint8_t> blob;
    std::vector<uint32_t> first16(static_cast<size_t>(hv.vocab_size) * 4 + 4, 0);
    for (uint32_t id = 0; id < hv.vocab_size; ++id) {
        off[id] = static_cast<uint32_t>(blob.size());
        if (id >= hv.token_bytes.size()) continue;
        const std::string& b = hv.token_bytes[id];
        blob.insert(blob.end(), b.begin(), b.end());
        std::memcpy(first16.data() + static_cast<size_t>(id) * 4, b.data(), b.size() < 16 ? b.size() : 16);
    }
    off[hv.vocab_size] = static_cast<uint32_t>(blob.size());
    blob.resize(blob.size() + 16);
    const uint32_t n_tiles = (n + gtok::kDecIds - 1) / gtok::kDecIds;
    std::vector<uint32_t> in(static_cast<size_t>(n) + 4 + gtok::kDecPer, 0);
    in[0] = n;
    if (n) std::memcpy(in.data() + 4, ids, static_cast<size_t>(n) * 4);
    std::vector<unsigned long long> st(n_tiles + 1, 0);
    std::vector<uint8_t> obuf(static_cast<size_t>(cap) + 32, 0xEE);
    uint8_t* o = obuf.data();
    o += (16 - (reinterpret_cast<uintptr_t>(o) & 15)) & 15;
    uint32_t ctl[16] = {0}, status[16] = {0};
    gtok::DecodeArgs a;
    std::memset(&a, 0, sizeof a);
    a.meta = in.data();
    a.ids = in.data() + 4;
    a.tok_off = off.data();
    a.blob = blob.data();
    a.tok16 = first16.data();
    a.vocab_size = hv.vocab_size;
    a.st = st.data();
    a.ctl = ctl;
    a.out = o;
    a.out_cap = cap;
    a.status = status;
    std::unique_ptr<gtok::DecodeSmem> sm(new gtok::DecodeSmem());
    CpuBlk blk;
    blk.reverse = reverse != 0;
    for (uint32_t t = 0; t < n_tiles; ++t) gtok::decode_tile(blk, a, *sm, static_cast<int>(t));
    if (err_bits) *err_bits = ctl[gtok::CTL_ERR];
    const uint32_t total = status[0];
    if (total <= cap && !(ctl[gtok::CTL_ERR] & gtok::kErrOutputFull)) {
        std::memcpy(out, o, total);
        // nothing may be written past the end
        for (uint32_t i = total; i < cap + 16 && o + i < obuf.data() + obuf.size(); ++i) if (o[i] != 0xEE) { if (err_bits) *err_bits |= 0x80000000u; break; }
    }
    return total;
}

// The normalisation kernel's table look-ups (hashed on the device side), one codepoint or pair at a time.
static gtok::DeviceTables nfc_lookup_tables(gtok::NfcWords& words) {
    gtok::nfc_table_words(words);
    gtok::DeviceTables tb;
    std::memset(&tb, 0, sizeof tb);
    tb.nfc_cp_hash = words.cp_hash.data(); tb.nfc_cp_hash_mask = static_cast<uint32_t>(words.cp_hash.size() / 2 - 1);
    tb.nfc_comp_hash = words.comp_hash.data(); tb.nfc_comp_hash_mask = static_cast<uint32_t>(words.comp_hash.size() / 4 - 1);
    tb.nfc_decomp = words.decomp.data(); tb.nfc_decomp_n = static_cast<uint32_t>(words.decomp.size() / 6);
    return tb;
}
// out[cp] = combining class | (number of codepoints in the full canonical decomposition, 0 = none) << 8, for cp < n
void gtok_emul_nfc_cp_info(uint32_t* out, uint32_t n) {
    gtok::NfcWords words;
    const gtok::DeviceTables tb = nfc_lookup_tables(words);
    for (uint32_t cp = 0; cp < n; ++cp) {
        const uint32_t info = cp >= 0xC0 ? gtok::nfc_cp_info(tb, cp) : 0u;
        out[cp] = gtok::nfc_ccc(tb, cp) | ((info >> 8) ? tb.nfc_decomp[6 * ((info >> 8) - 1) + 1] << 8 : 0u);
    }
}
void gtok_emul_nfc_compose(const uint32_t* first, const uint32_t* second, uint32_t* out, uint32_t n) {
    gtok::NfcWords words;
    const gtok::DeviceTables tb = nfc_lookup_tables(words);
    for (uint32_t i = 0; i < n; ++i) out[i] = gtok::nfc_compose(tb, first[i], second[i]);
}

// The bit scans the whitespace and newline walks use inside a tile's window, on planes the caller makes up:
// s, cr: one bit per byte (16 bits per entry, entries in eight-byte aligned rows), doc: 32 bits per word.
int gtok_emul_plain_ws_end(const uint16_t* s, const uint16_t* cr, const uint32_t* doc, int i, int i_end) {
    return gtok::plain_ws_end(s, cr, doc, i, i_end);
}
int gtok_emul_newline_run_begin(const uint16_t* cr, const uint32_t* doc, int i, int i_begin) {
    return gtok::newline_run_begin(cr, doc, i, i_begin);
}

int gtok_emul_plan_chunks(void* h, const uint8_t* text, uint64_t len, uint32_t n_parts, uint64_t* out) {
    std::vector<uint64_t> cuts;
    gtok::plan_chunks(static_cast<Emul*>(h)->hv, text, len, n_parts, cuts);
    std::memcpy(out, cuts.data(), cuts.size() * sizeof(uint64_t));
    return 0;
}

}  // extern "C"
