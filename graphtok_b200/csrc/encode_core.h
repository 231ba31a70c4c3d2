// The encode path, tile by tile (4096 bytes of text): pre-tokenization (boundary bits),
// per-pre-token BPE merging and output assembly.  The tile programs, one per kernel:
//
//   pretok_tile   : text bytes -> one boundary bit per byte (a set bit = a pre-token starts
//                   here) plus one "added token starts here" bit; added-token ids go straight
//                   to their slots.
//   words_tile    : every pre-token of the tile against the whole-word table; known ones get
//                   their id in the tile's slot array (one u32 per byte, id at the byte where the
//                   pre-token starts), unknown ones go to global lists by length class.
//   miss_batch    : a batch of unknown pre-tokens of one length class: greedy merge loop, one
//                   thread per pre-token, over a shared-memory symbol arena.
//   long_word     : one pre-token of more than 64 bytes, by a whole block (run-length merge for
//                   runs of one character, round-batched merge otherwise).
//   assemble_tile : the tile's slots -> ids at their final place in the output.
//
// All are written against a small "thread block" interface (Blk):
//     blk.par(f)                run f(tid) for every thread, then barrier
//     blk.excl_scan(arr,total)  in-place exclusive scan of arr[kThreads]
//     blk.lookback(st,tile,total,ctl)  publish this tile's total, return the sum of all earlier tiles'
// so that the CUDA kernels in encode_kernels.cu (one real thread per tid) and a
// serial emulation used by the CPU tests execute the very same logic.  Nothing
// outside a par() body may depend on the order in which tids run, and no par()
// body may read what another tid writes in the same par().
//
// Reference for behaviour (not structure): the boundary predicates restate the
// regular expressions' semantics as the reference does in
// src/pretok_boundary.h:221-297 (GPT-2) and :511-671 (Llama-3 / Qwen2.5), in the
// byte domain instead of over dense codepoint arrays; the merge loop is the
// greedy lowest-rank-first rule of src/tokenizer.cu:360-580 / src/host_encode.cc:617-648;
// the batched rounds for long pre-tokens follow the idea of src/tokenizer.cu:754-791.
#pragma once
#include <stdint.h>

#include "device_tables.h"

#if defined(__CUDACC__)
#define GTOK_DEV __device__ __forceinline__
#define GTOK_DEV_NOINLINE static __device__ __noinline__
#else
#define GTOK_DEV inline
#define GTOK_DEV_NOINLINE inline
#endif

namespace gtok {

constexpr int kTile = 4096;        // bytes per tile
constexpr int kThreads = 256;      // threads per block
constexpr int kPer = kTile / kThreads;   // 16 bytes per thread
constexpr int kHaloL = 128;
constexpr int kHaloR = 64;
constexpr int kWin = kHaloL + kTile + kHaloR;
constexpr int kTileWords = kTile / 32;
// Pre-tokenization works on tiles of its own: a window of two 16-byte chunks per thread (halos
// included), so that every thread has the same work in the chunk phases and a document of up to
// about 4.7 MB is a single wave of blocks on a B200.
constexpr int kPChunks = 2 * kThreads;
constexpr int kPWin = kPChunks * 16;                    // 8192 bytes staged per tile
constexpr int kPTile = kPWin - kHaloL - kHaloR;         // 8000 bytes of text per tile
constexpr int kPTileWords = kPTile / 32;                // 250 mask words per tile
constexpr int kLitPlaces = 48;                          // places per tile where an added-token literal may start, looked up in parallel
constexpr int kUcStage1Bmp = 512;        // first-stage entries of the class table that cover U+0000..U+FFFF (128 codepoints each)
constexpr int kUcStage2Words = 1664;     // words of its second stage (unicode_class_table.h; checked where the tables are uploaded)

// Diagnostics (contexts created with GTOK_PHASE_CLOCKS set): 32 phase counters, then for each of the
// four kernels and each of its first kTlBlocks blocks kTlSlots nanosecond stamps of the GPU's global
// timer: [0] block started, [1] block finished, [2..] its first work items finished.
constexpr int kPhaseWords = 32;
constexpr int kTlBlocks = 1280;
constexpr int kTlSlots = 8;
constexpr int kTlWords = 6 * kTlBlocks * kTlSlots;     // table 4: end of each phase of a block's first pre-tokenization tile, then (overwritten by the later kernel) of its last miss batch; table 5: the single-block kernel's stages

constexpr uint32_t kInvalidTok = 0xFFFFFFFFu;
constexpr uint32_t kLongRef = 0x80000000u;      // tok[] entry that stands for a whole long pre-token
constexpr uint32_t kDirty = 0xFFFFFFFEu;
constexpr uint32_t kReprobe = 0xFFFFFFFEu;

constexpr int kMedWordMax = 64;      // longest pre-token merged by a single thread
constexpr int kTokExtra = 64;        // token slots past the tile for pre-tokens that start in it

// Error bits accumulated in ctl[2] and reported to the host.
enum : uint32_t {
    kErrOutputFull = 1u,      // more tokens than the output buffer holds
    kErrWaitExpired = 2u,     // a look-back wait gave up
    kErrProbeLimit = 4u,      // a table probe ran past its limit (corrupt table)
    kErrInternal = 8u,
    kErrNfcLong = 16u,        // a stretch to normalise holds more codepoints than one thread takes
    kErrNfcFull = 32u,        // the normalised text does not fit the text buffer
};

// Per-byte attribute (shared memory, pretok only).
enum : uint8_t {
    A_L = 0, A_N = 1, A_S = 2, A_O = 3, A_CONT = 4, A_ADDED = 5, A_P = 6, A_OUT = 7, A_CLS = 7,
    A_CRLF = 8, A_SP = 16, A_DOC = 32, A_CJK = 64,
};
// A_P (\p{P} or \p{S}) and A_CJK (the three ranges of the second DeepSeek-V3 pattern) only occur with
// the wide class table, where A_L also covers \p{M}.

// Class of codepoint cp from the two-stage table: two bits per codepoint, eight words per leaf
// (L, N, S, other), or with `wide` four bits per codepoint, sixteen words per leaf (the values of
// A_L, A_N, A_S, A_O, A_P).
template <class Stage1, class Stage2>
GTOK_DEV uint32_t uc_class(Stage1 s1, Stage2 s2, uint32_t cp, bool wide) {
    if (cp > 0x10FFFFu) return A_O;
    const uint32_t leaf = s1(cp >> 7);
    if (wide) return (s2(leaf * 16u + ((cp & 127u) >> 3)) >> ((cp & 7u) * 4u)) & 15u;
    return (s2(leaf * 8u + ((cp & 127u) >> 4)) >> ((cp & 15u) * 2u)) & 3u;
}
GTOK_DEV bool cp_is_cjk(uint32_t cp) { return (cp >= 0x4E00u && cp <= 0x9FA5u) || (cp >= 0x3040u && cp <= 0x30FFu); }

struct EncodeArgs {
    const uint8_t* text;          // padded; readable kTile + kWin bytes past the capacity
    const uint32_t* meta;         // [0] = n_bytes, [1] = n_docs
    const uint32_t* doc_off;      // [n_docs + 1] byte offsets (batch) or nullptr
    const uint32_t* docmask;      // one bit per byte, set at document starts (batch) or nullptr
    uint32_t* bmask;              // boundary bits, 1 per byte
    uint32_t* amask;              // added-token-start bits
    uint32_t* tile_nb;            // boundaries per tile
    uint32_t one_list;            // single-block kernel: every unknown pre-token of 2..64 bytes goes to the one list gmiss, whatever its length
    uint32_t sum_tiles;           // documents of up to this many tiles get their tile bases by direct summation (kSumTiles; tests use 0)
    uint32_t* tile_tok;           // ids per tile (by the tile where their pre-token starts): set by words, added to by miss, summed by assemble
    unsigned long long* st1;      // pretok look-back state per tile
    unsigned long long* st2;      // merge look-back state per tile
    uint32_t* ctl;                // [0] pretok ticket, [1] assemble ticket, [2] error bits, [3] exit counter,
                                  // [4] unknown pre-tokens, [5] long pre-tokens, [6] batch ticket, [7] long ticket
    uint32_t* gstage;             // u32 per byte: ids of long pre-tokens
    uint32_t* gwork_rk;           // u32 per byte: rank workspace for very long pre-tokens
    uint32_t* gwork_nw;           // u32 per byte: result workspace for very long pre-tokens
    uint32_t* stage;              // u32 per byte: id stored at the byte where its pre-token starts (+k for its k-th id), else invalid
    uint32_t* ovf;                // kTokExtra u32 per tile: ids of a tile's last pre-token that do not fit before the tile's end
    unsigned long long* gmiss;    // pre-tokens of 2..16 bytes the whole-word table did not know: position | len << 32
    unsigned long long* gmed;     // the same for 33..64 bytes (from the front) and 17..32 bytes (from the back, downwards)
    uint32_t gmed_cap;            // entries in gmed
    unsigned long long* gmed1;    // the same for 33..48 bytes
    uint32_t* glong_g;            // pre-tokens longer than 64 bytes: position, length (0 = not known yet), id count
    uint32_t* glong_len;
    uint32_t* glong_cnt;
    uint32_t* out_tokens;
    uint32_t out_cap;
    uint32_t* out_doc_tok;        // [n_docs + 1] token offsets (batch) or nullptr
    uint32_t* status;             // [0] total tokens, [1] error bits (host-visible)
    unsigned long long* phase_clk; // optional: cycles spent per phase, summed over blocks (diagnostics); from word kPhaseWords on, the block timeline
    // Normalisation (vocabularies that declare NFC); raw == nullptr otherwise.
    const uint8_t* raw;           // text as the caller gave it, padded like `text`
    const uint32_t* raw_meta;     // [0] = bytes, [1] = documents, [2] = 1 when the text is normalised already
    const uint32_t* raw_doc_off;  // [n_docs + 1] offsets into raw (batch) or nullptr
    const uint32_t* raw_docmask;  // document-start bits over raw (batch) or nullptr
    uint8_t* norm_text;           // = text, writable
    uint32_t* norm_meta;          // = meta, writable
    uint32_t* norm_doc_off;       // = doc_off, writable
    unsigned long long* st0;      // normalisation look-back state per tile
    uint32_t text_cap;            // bytes the text buffer holds
    DeviceTables tb;
};

// ---- small portable helpers ---------------------------------------------------
// Loads of data a kernel only reads go through the non-coherent path.  A translation unit whose
// kernel reads what it wrote itself (the single-block kernel, which runs all tile programs one after
// the other) defines GTOK_COHERENT_LOADS before including this header: every such load is then an
// ordinary one, which sees the block's own earlier stores after a barrier.
template <class T>
GTOK_DEV T ldg(const T* p) {
#if defined(__CUDA_ARCH__) && !defined(GTOK_COHERENT_LOADS)
    return __ldg(p);
#else
    return *p;
#endif
}
#if defined(__CUDA_ARCH__)
__device__ __forceinline__ uint4 ld128(const uint4* p) {       // text and slots: written by the same kernel in the single-block case
#if defined(GTOK_COHERENT_LOADS)
    return *p;
#else
    return __ldg(p);
#endif
}
#endif
GTOK_DEV int popc32(uint32_t x) {
#if defined(__CUDA_ARCH__)
    return __popc(x);
#else
    return __builtin_popcount(x);
#endif
}
GTOK_DEV int ffs32(uint32_t x) {   // index of lowest set bit, x != 0
#if defined(__CUDA_ARCH__)
    return __ffs(x) - 1;
#else
    return __builtin_ctz(x);
#endif
}
GTOK_DEV int fls32(uint32_t x) {   // index of highest set bit, x != 0
#if defined(__CUDA_ARCH__)
    return 31 - __clz(x);
#else
    return 31 - __builtin_clz(x);
#endif
}
GTOK_DEV uint64_t brev64(uint64_t x) {
#if defined(__CUDA_ARCH__)
    return __brevll(x);
#else
    x = ((x >> 1) & 0x5555555555555555ull) | ((x & 0x5555555555555555ull) << 1);
    x = ((x >> 2) & 0x3333333333333333ull) | ((x & 0x3333333333333333ull) << 2);
    x = ((x >> 4) & 0x0F0F0F0F0F0F0F0Full) | ((x & 0x0F0F0F0F0F0F0F0Full) << 4);
    return __builtin_bswap64(x);
#endif
}
GTOK_DEV uint32_t shared_add(uint32_t* p, uint32_t v) {
#if defined(__CUDA_ARCH__)
    return atomicAdd(p, v);
#else
    uint32_t o = *p; *p = o + v; return o;
#endif
}
GTOK_DEV void shared_or(uint32_t* p, uint32_t v) {
#if defined(__CUDA_ARCH__)
    atomicOr(p, v);
#else
    *p |= v;
#endif
}
GTOK_DEV void shared_max64(unsigned long long* p, unsigned long long v) {
#if defined(__CUDA_ARCH__)
    atomicMax(p, v);
#else
    if (v > *p) *p = v;
#endif
}
GTOK_DEV void global_or(uint32_t* p, uint32_t v) {
#if defined(__CUDA_ARCH__)
    atomicOr(p, v);
#else
    *p |= v;
#endif
}
GTOK_DEV void global_add(uint32_t* p, uint32_t v) {
#if defined(__CUDA_ARCH__)
    atomicAdd(p, v);
#else
    *p += v;
#endif
}
GTOK_DEV unsigned long long load_state(const unsigned long long* p) {
#if defined(__CUDA_ARCH__)
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
#else
    return *p;
#endif
}
GTOK_DEV void store_state(unsigned long long* p, unsigned long long v) {
#if defined(__CUDA_ARCH__)
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
    *p = v;
#endif
}
GTOK_DEV unsigned long long cycle_now() {
#if defined(__CUDA_ARCH__)
    return clock64();
#else
    return 0;
#endif
}
GTOK_DEV void add_cycles(unsigned long long* p, unsigned long long v) {
#if defined(__CUDA_ARCH__)
    atomicAdd(p, v);
#else
    *p += v;
#endif
}
GTOK_DEV void backoff() {
#if defined(__CUDA_ARCH__)
    __nanosleep(40);
#endif
}

constexpr unsigned long long kStAgg = 1ull << 62;     // value covers this tile only
constexpr unsigned long long kStFinal = 2ull << 62;   // value needs nothing from earlier tiles
constexpr int kWaitLimit = 1 << 22;                   // polls before a wait gives up

// Waits for tile j's state to be published.  Returns 0 (and raises the error
// bit) when the limit runs out, which the host reports as a failed call.
GTOK_DEV unsigned long long wait_state(const unsigned long long* st, int j, uint32_t* ctl) {
    for (int it = 0; it < kWaitLimit; ++it) {
        unsigned long long v = load_state(st + j);
        if (v >> 62) return v;
        backoff();
    }
    global_or(ctl + 2, kErrWaitExpired);
    return kStFinal;
}

// Counts one more finished producer, after everything this block wrote before (the caller has
// passed a block barrier since).
GTOK_DEV void release_add(uint32_t* p, uint32_t v) {
#if defined(__CUDA_ARCH__)
    __threadfence();
    atomicAdd(p, v);
#else
    *p += v;
#endif
}
// Waits until the counter reaches `want`; false (and the error bit) when the limit runs out.
GTOK_DEV bool wait_count(const uint32_t* p, uint32_t want, uint32_t* ctl) {
    for (int it = 0; it < kWaitLimit; ++it) {
#if defined(__CUDA_ARCH__)
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
#else
        const uint32_t v = *p;
#endif
        if (v >= want) return true;
        backoff(); backoff(); backoff(); backoff();       // many blocks poll this one word
    }
    global_or(ctl + 2, kErrWaitExpired);
    return false;
}

// ---- merge-rule probe ----------------------------------------------------------
struct RankRes { uint32_t rank, res; };
#if defined(__CUDA_ARCH__)
// Both slots of a bucket with one 256-bit load (sm_100): the merge kernel is bound by the number of
// scattered load requests its threads make, and this halves them.
__device__ __forceinline__ void load_bucket(const MergeSlot* bucket, uint4* s0, uint4* s1) {
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(s0->x), "=r"(s0->y), "=r"(s0->z), "=r"(s0->w), "=r"(s1->x), "=r"(s1->y), "=r"(s1->z), "=r"(s1->w)
                 : "l"(bucket));
}
#endif
// A rule is in its first bucket (two slots, one 32-byte sector, read with one 256-bit load) unless that
// bucket's flag says some rule went to its second bucket; only then is the second bucket read as well.
GTOK_DEV RankRes probe_rule(const DeviceTables& tb, uint32_t l, uint32_t r) {
    uint32_t b1, b2;
    merge_buckets(l, r, tb.merge_shift, &b1, &b2);
#if defined(__CUDA_ARCH__)
    uint4 s0, s1;
    load_bucket(tb.merge + 2 * b1, &s0, &s1);
    if (s0.x == l && s0.y == r) return RankRes{s0.z, s0.w & ~kBucketSpills};
    if (s1.x == l && s1.y == r) return RankRes{s1.z, s1.w};
    if (s0.w & kBucketSpills) {
        uint4 u0, u1;
        load_bucket(tb.merge + 2 * b2, &u0, &u1);
        if (u0.x == l && u0.y == r) return RankRes{u0.z, u0.w & ~kBucketSpills};
        if (u1.x == l && u1.y == r) return RankRes{u1.z, u1.w};
    }
#else
    for (int pass = 0; pass < 2; ++pass) {
        const uint32_t b = pass ? b2 : b1;
        const MergeSlot& s0 = tb.merge[2 * b];
        const MergeSlot& s1 = tb.merge[2 * b + 1];
        if (s0.left == l && s0.right == r) return RankRes{s0.rank, s0.result & ~kBucketSpills};
        if (s1.left == l && s1.right == r) return RankRes{s1.rank, s1.result};
        if (pass == 0 && !(tb.merge[2 * b1].result & kBucketSpills)) break;
    }
#endif
    return RankRes{kNoRank, 0};
}

// Probe chain of a key from slot h on (h = its home slot, or further along when the caller has
// looked at the slots before).
GTOK_DEV uint32_t probe_word_from(const DeviceTables& tb, uint64_t k0, uint64_t k1, uint32_t h) {
    for (int i = 0; i < kProbeLimit; ++i) {
#if defined(__CUDA_ARCH__)
        const uint4* sp = reinterpret_cast<const uint4*>(tb.word + h);
        uint4 a = __ldg(sp);
        uint4 b = __ldg(sp + 1);
        uint64_t s0 = (static_cast<uint64_t>(a.y) << 32) | a.x, s1 = (static_cast<uint64_t>(a.w) << 32) | a.z;
        uint32_t id = b.x;
#else
        uint64_t s0 = tb.word[h].k0, s1 = tb.word[h].k1;
        uint32_t id = tb.word[h].id;
#endif
        if (id == kNoToken) return kNoToken;
        if (s0 == k0 && s1 == k1) return id;
        h = (h + 1) & tb.word_mask;
    }
    return kNoToken;
}
GTOK_DEV uint32_t probe_word(const DeviceTables& tb, uint64_t k0, uint64_t k1) {
    return probe_word_from(tb, k0, k1, word_hash(k0, k1) & tb.word_mask);
}

// Whole pre-token of 16 bytes or more, present in the vocabulary?  (ignore_merges)
GTOK_DEV uint32_t probe_long(const DeviceTables& tb, const uint8_t* text, uint32_t g, uint32_t len) {
    if (len > tb.long_max_len) return kNoToken;
    uint64_t h = kLongHashSeed;
    for (uint32_t i = 0; i < len; ++i) h = long_hash_step(h, ldg(text + g + i));
    h = long_hash_finish(h, len);
    uint32_t at = static_cast<uint32_t>(h) & tb.long_mask;
    for (int i = 0; i < kProbeLimit; ++i) {
        LongSlot s = tb.longtab[at];
        if (s.id == kNoToken) return kNoToken;
        if (s.hash == h && s.len == len) {
            bool same = true;
            for (uint32_t k = 0; k < len && same; ++k) same = ldg(tb.long_blob + s.off + k) == ldg(text + g + k);
            if (same) return s.id;
        }
        at = (at + 1) & tb.long_mask;
    }
    return kNoToken;
}

// Same lookup with the bytes at hand (shared memory).  The spellings in long_blob start on 4-byte
// boundaries and are zero padded to one, so a candidate is compared a word at a time, all its
// words requested together.
GTOK_DEV uint32_t probe_long_bytes(const DeviceTables& tb, const uint8_t* bytes, uint32_t len) {
    if (len > tb.long_max_len) return kNoToken;
    uint64_t h = kLongHashSeed;
    for (uint32_t i = 0; i < len; ++i) h = long_hash_step(h, bytes[i]);
    h = long_hash_finish(h, len);
    uint32_t at = static_cast<uint32_t>(h) & tb.long_mask;
    for (int i = 0; i < kProbeLimit; ++i) {
        LongSlot s = tb.longtab[at];
        if (s.id == kNoToken) return kNoToken;
        if (s.hash == h && s.len == len) {
            uint32_t diff = 0;
            for (uint32_t k = 0; k < len; k += 4) {
                const uint32_t bw = ldg(reinterpret_cast<const uint32_t*>(tb.long_blob + s.off + k));
                uint32_t tw = 0;
                for (uint32_t b = 0; b < 4 && k + b < len; ++b) tw |= static_cast<uint32_t>(bytes[k + b]) << (8 * b);
                diff |= bw ^ tw;
            }
            if (!diff) return s.id;
        }
        at = (at + 1) & tb.long_mask;
    }
    return kNoToken;
}

// Two independent rule probes whose first-bucket loads are all issued before the first compare, so
// that the pair costs one memory round trip (a second one for a probe whose bucket is flagged).
GTOK_DEV void probe_rule2(const DeviceTables& tb, bool want1, uint32_t l1, uint32_t r1, RankRes* o1,
                          bool want2, uint32_t l2, uint32_t r2, RankRes* o2) {
    *o1 = RankRes{kNoRank, 0};
    *o2 = RankRes{kNoRank, 0};
#if defined(__CUDA_ARCH__)
    uint32_t a1, a2, b1, b2;
    merge_buckets(l1, r1, tb.merge_shift, &a1, &a2);
    merge_buckets(l2, r2, tb.merge_shift, &b1, &b2);
    uint4 x0 = make_uint4(kEmptyKey, 0, 0, 0), x1 = x0, y0 = x0, y1 = x0;
    if (want1) load_bucket(tb.merge + 2 * a1, &x0, &x1);
    if (want2) load_bucket(tb.merge + 2 * b1, &y0, &y1);
    if (want1) {
        if (x0.x == l1 && x0.y == r1) *o1 = RankRes{x0.z, x0.w & ~kBucketSpills};
        else if (x1.x == l1 && x1.y == r1) *o1 = RankRes{x1.z, x1.w};
        else if (x0.w & kBucketSpills) {
            uint4 u0, u1;
            load_bucket(tb.merge + 2 * a2, &u0, &u1);
            if (u0.x == l1 && u0.y == r1) *o1 = RankRes{u0.z, u0.w & ~kBucketSpills};
            else if (u1.x == l1 && u1.y == r1) *o1 = RankRes{u1.z, u1.w};
        }
    }
    if (want2) {
        if (y0.x == l2 && y0.y == r2) *o2 = RankRes{y0.z, y0.w & ~kBucketSpills};
        else if (y1.x == l2 && y1.y == r2) *o2 = RankRes{y1.z, y1.w};
        else if (y0.w & kBucketSpills) {
            uint4 u0, u1;
            load_bucket(tb.merge + 2 * b2, &u0, &u1);
            if (u0.x == l2 && u0.y == r2) *o2 = RankRes{u0.z, u0.w & ~kBucketSpills};
            else if (u1.x == l2 && u1.y == r2) *o2 = RankRes{u1.z, u1.w};
        }
    }
#else
    if (want1) *o1 = probe_rule(tb, l1, r1);
    if (want2) *o2 = probe_rule(tb, l2, r2);
#endif
}

// ---- document-start bits ---------------------------------------------------------
GTOK_DEV bool is_docstart_global(const EncodeArgs& a, int p) {
    if (p == 0) return true;
    if (!a.docmask) return false;
    return (ldg(a.docmask + (p >> 5)) >> (p & 31)) & 1u;
}
// The two pointers the raw-byte walks need, by value: a walk that runs in a function of its own would otherwise
// fetch them through the argument block's address at every step.
struct RawText {
    const uint8_t* text;
    const uint32_t* docmask;
};
GTOK_DEV RawText raw_text(const EncodeArgs& a) { return RawText{a.text, a.docmask}; }
GTOK_DEV bool raw_docstart(RawText t, int p) {
    if (p == 0) return true;
    if (!t.docmask) return false;
    return (ldg(t.docmask + (p >> 5)) >> (p & 31)) & 1u;
}

// ==================================================================================
//                                   PRE-TOKENIZATION
// ==================================================================================
// One-hot byte used to build bit planes: bit c for class c (L,N,S,O,CONT,ADDED), then flags.
enum : uint8_t { kOhL = 1, kOhN = 2, kOhS = 4, kOhO = 8, kOhC = 16, kOhAdded = 32, kOhCrlf = 64, kOhSp = 128 };
enum { PL_L = 0, PL_N, PL_S, PL_O, PL_C, PL_AD, PL_CRLF, PL_SP, PL_AP, kPlanes };

GTOK_DEV uint8_t onehot_of(uint8_t at) {
    int c = at & A_CLS;
    if (c == A_P) c = A_O;        // the planes know four classes; the wide classes are read from the attribute bytes
    uint8_t oh = c <= A_ADDED ? static_cast<uint8_t>(1u << c) : 0;
    if (at & A_CRLF) oh |= kOhCrlf;
    if (at & A_SP) oh |= kOhSp;
    return oh;
}
// Bit k of each of the four bytes of w, gathered into the low four bits.
GTOK_DEV uint32_t gather_bit4(uint32_t w, int k) { return (((w >> k) & 0x01010101u) * 0x01020408u) >> 24; }

struct PretokSmem {
    alignas(16) uint8_t txt[kPWin + 16];
    alignas(16) uint8_t attr[kPWin + 16];
    alignas(16) uint8_t oh[kPWin + 16];       // one-hot class + flags per byte (see kOh*)
    alignas(8) uint16_t plane[kPlanes][kPWin / 16 + 4];   // bit planes of the window, 16 bytes per entry
    uint32_t lut[256];                       // byte -> attr | one-hot << 8 | (opens an added-token literal) << 16: ASCII as classified, continuation bytes, lead bytes as "other" until decoded
    uint16_t cand16[kPWin / 16 + 4];          // per 16-byte chunk: bytes that open an added-token literal
    alignas(16) uint16_t ucs1[kUcStage1Bmp]; // the class table's first stage for the BMP and its whole second stage, copied once per block
    alignas(16) uint32_t ucs2[kUcStage2Words];
    uint32_t lit_lens[kLitLens];             // the distinct added-token literal lengths (copy of the tables')
    unsigned long long lit_best[kLitPlaces]; // per listed place: longest literal found there, length << 32 | id
    uint16_t lit_at[kLitPlaces];             // places of the tile's window where a literal may start
    uint32_t dirty[(kPWin / 16 + 31) / 32];   // chunks whose plane entries a painted literal has made stale
    uint32_t dsw[kPWin / 32 + 2];             // document-start bits of the window
    uint16_t bnd16[2 * kPTileWords + 4], add16[2 * kPTileWords + 4], pend16[2 * kPTileWords + 4];
    uint16_t lead16[2 * kPTileWords + 4], nlead16[2 * kPTileWords + 4], nstart16[2 * kPTileWords + 4];
    uint32_t carry[kPTileWords + 8];
    uint32_t sum_has[32], sum_cnt[32], lane_last[32], lane_firstn[32];
    uint32_t scan[kThreads];
    uint32_t misc[8];
    int far_run[4];                          // runs that leave the window, found by the whole block before the rules are applied: {position the forward walk starts at, its answer, position the backward walk starts at, its answer}
    unsigned long long clk_last;
};

// With the wide class table (DeepSeek-V3) the block's copy of the narrow table is not used, and its
// room holds four more planes: punctuation and symbols, ASCII letters, ASCII punctuation, and the lead
// bytes of codepoints inside the three CJK ranges.
enum { XP_PS = 0, XP_AL, XP_APU, XP_CJK, kXPlanes };
constexpr int kXPlaneStride = kPWin / 16 + 8;
static_assert(kXPlanes * kXPlaneStride * 2 <= kUcStage2Words * 4, "the extra planes fit the class-table copy");
GTOK_DEV uint16_t* xplane(PretokSmem& sm, int k) { return reinterpret_cast<uint16_t*>(sm.ucs2) + k * kXPlaneStride; }
GTOK_DEV const uint16_t* xplane(const PretokSmem& sm, int k) { return reinterpret_cast<const uint16_t*>(sm.ucs2) + k * kXPlaneStride; }
// Their entries of chunk c from its attribute bytes and its text.
GTOK_DEV void chunk_xplanes(PretokSmem& sm, int c, const uint32_t* aw, const uint32_t* tw) {
    uint32_t ps = 0, al = 0, asc = 0, cjk = 0;
    for (int j = 0; j < 4; ++j) {
        const uint32_t x = (aw[j] & 0x07070707u) ^ (A_P * 0x01010101u);            // a zero byte: class A_P
        const uint32_t zp = ~(((x & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | x) & 0x80808080u;
        ps |= gather_bit4(zp, 7) << (4 * j);
        cjk |= gather_bit4(aw[j], 6) << (4 * j);
        const uint32_t t = tw[j];
        const uint32_t lo7 = (t | 0x20202020u) & 0x7F7F7F7Fu;                       // letters folded to lower case
        const uint32_t ge_a = lo7 + (0x80u - 'a') * 0x01010101u, gt_z = lo7 + (0x80u - 'z' - 1u) * 0x01010101u;
        al |= gather_bit4(ge_a & ~gt_z & ~t, 7) << (4 * j);
        asc |= gather_bit4(~t, 7) << (4 * j);
    }
    xplane(sm, XP_PS)[c] = static_cast<uint16_t>(ps);
    xplane(sm, XP_AL)[c] = static_cast<uint16_t>(al);
    xplane(sm, XP_APU)[c] = static_cast<uint16_t>(ps & asc);
    xplane(sm, XP_CJK)[c] = static_cast<uint16_t>(cjk);
}

// The nine plane entries of 16-byte chunk c from its one-hot bytes and its text.
GTOK_DEV void chunk_planes(PretokSmem& sm, int c, const uint32_t* ow, const uint32_t* tw) {
    for (int k = 0; k < 8; ++k)
        sm.plane[k][c] = static_cast<uint16_t>(gather_bit4(ow[0], k) | (gather_bit4(ow[1], k) << 4) | (gather_bit4(ow[2], k) << 8) | (gather_bit4(ow[3], k) << 12));
    uint32_t ap = 0;
    for (int j = 0; j < 4; ++j) {
        uint32_t x = tw[j] ^ 0x27272727u;                      // a zero byte marks an apostrophe
        uint32_t z = (x - 0x01010101u) & ~x & 0x80808080u;
        // the borrow trick can flag a byte above a true zero; apostrophes are rare, so check exactly
        if (z) for (int k = 0; k < 4; ++k) if (((tw[j] >> (8 * k)) & 0xFFu) == 0x27u) ap |= 1u << (j * 4 + k);
    }
    sm.plane[PL_AP][c] = static_cast<uint16_t>(ap);
}

// View of one tile's window for the predicate code.
struct Win {
    const PretokSmem* sm;
    const EncodeArgs* a;
    int lo;        // global position of window byte 0 (may be negative)
    int vlo, vhi;  // positions in [vlo, vhi) have a trustworthy shared-memory attribute
    int n;
};

// Longest added-token literal starting at global position s, clamped to the
// document of s.  Returns its byte length (0 = none) and its id.
template <class GetByte>
GTOK_DEV uint32_t match_literal(const EncodeArgs& a, int s, int n, GetByte byte_at, uint32_t* id_out) {
    const DeviceTables& tb = a.tb;
    uint32_t node = ldg(tb.trie_root + byte_at(s));
    if (node == kNoToken) return 0;
    uint32_t best = 0;
    int q = s + 1;
    for (;;) {
        // the node's skip string: bytes that must follow before the node itself is reached
        const uint32_t sk = ldg(tb.trie_skip + node);
        bool off_path = false;
        for (uint32_t j = 0, len = sk & 0xFFu; j < len; ++j, ++q) {
            if (q >= n || static_cast<uint32_t>(q - s) >= tb.added_max_bytes || (a.docmask && is_docstart_global(a, q)) ||
                byte_at(q) != ldg(tb.trie_blob + (sk >> 8) + j)) { off_path = true; break; }
        }
        if (off_path) break;
        uint32_t term = ldg(tb.trie_terminal + node);
        if (term != kNoToken) { best = static_cast<uint32_t>(q - s); *id_out = term; }
        if (q >= n || static_cast<uint32_t>(q - s) >= tb.added_max_bytes) break;
        if (a.docmask && is_docstart_global(a, q)) break;
        uint32_t want = byte_at(q);
        uint32_t first = ldg(tb.trie_first + node), cnt = ldg(tb.trie_count + node);
        uint32_t next = kNoToken;
        for (uint32_t e = 0; e < cnt; ++e) {
            uint32_t ed = ldg(tb.trie_edges + first + e);
            if ((ed & 0xFF) == want) { next = ed >> 8; break; }
        }
        if (next == kNoToken) break;
        node = next;
        ++q;
    }
    return best;
}

// The same answer from the hashed literal table (device_tables.h): the text's hash at every length
// some literal has, one slot read per length, and a slot whose hash and length agree compared with
// the text four bytes at a time.  The longest confirmed literal wins.  Everything stays in registers.
struct LitView {                 // what the hashed matcher needs, by value (lens may point to shared memory)
    const LitSlot* tab;
    const uint32_t* lens;
    uint32_t mask, n_lens, max_bytes;
};
// Is the literal of length `len` whose weighted byte sum is h (see lit_hash_finish) in the table, and
// does it spell the text at s?  Returns its id or kNoToken.
template <class GetByte>
GTOK_DEV uint32_t lit_lookup(const LitView& lv, uint32_t h, uint32_t len, int s, GetByte byte_at) {
    const uint32_t hf = lit_hash_finish(h, len);
    uint32_t at = hf & lv.mask;
    for (int i = 0; i < kProbeLimit; ++i) {
        const LitSlot* sl = lv.tab + at;
        const uint32_t id = ldg(&sl->id);
        if (id == kNoToken) return kNoToken;
        if (ldg(&sl->hash) == hf && ldg(&sl->len) == len) {
            uint32_t diff = 0;
            for (uint32_t j = 0; j < len; j += 4) {
                const uint32_t lw = ldg(reinterpret_cast<const uint32_t*>(sl->bytes + j));
                uint32_t tw = 0;
                for (uint32_t b = 0; b < 4 && j + b < len; ++b) tw |= byte_at(s + static_cast<int>(j + b)) << (8 * b);
                diff |= lw ^ tw;
            }
            if (!diff) return id;
        }
        at = (at + 1) & lv.mask;
    }
    return kNoToken;
}
// Bytes a literal at s may span: up to the end of the text, of the document, and the longest literal.
template <class IsDoc>
GTOK_DEV uint32_t lit_limit(const LitView& lv, bool batch, int s, int n, IsDoc is_doc) {
    uint32_t limit = static_cast<uint32_t>(n - s);
    if (limit > lv.max_bytes) limit = lv.max_bytes;
    if (batch) for (uint32_t k = 1; k < limit; ++k) if (is_doc(s + static_cast<int>(k))) { limit = k; break; }
    return limit;
}
// The longest literal at s, one thread: one pass over the bytes, a look-up at every literal length.
template <class GetByte, class IsDoc>
GTOK_DEV uint32_t match_literal_hashed(const LitView& lv, bool batch, int s, int n, GetByte byte_at, IsDoc is_doc, uint32_t* id_out) {
    const uint32_t limit = lit_limit(lv, batch, s, n, is_doc);
    uint32_t best = 0, li = 0, h = 0, pk = kLitHashK;
    uint32_t next_len = lv.lens[0];
    for (uint32_t len = 1; len <= limit; ++len) {
        h += byte_at(s + static_cast<int>(len) - 1) * pk;
        pk *= kLitHashK;
        if (len != next_len) continue;
        const uint32_t id = lit_lookup(lv, h, len, s, byte_at);
        if (id != kNoToken) { best = len; *id_out = id; }
        if (++li >= lv.n_lens) break;
        next_len = lv.lens[li];
    }
    return best;
}
template <class GetByte>
GTOK_DEV uint32_t longest_literal(const EncodeArgs& a, int s, int n, GetByte byte_at, uint32_t* id_out) {
    if (!a.tb.lit_n_lens) return match_literal(a, s, n, byte_at, id_out);
    const LitView lv{a.tb.littab, a.tb.lit_lens, a.tb.lit_mask, a.tb.lit_n_lens, a.tb.added_max_bytes};
    return match_literal_hashed(lv, a.docmask != nullptr, s, n, byte_at, [&](int q) { return is_docstart_global(a, q); }, id_out);
}

// The literal at global position s as seen from a tile's window (text bytes in shared memory from
// global position lo on, the rest from global memory).  A function of its own, not inlined: it runs
// for a handful of bytes per tile and must not cost the tile program registers; everything it
// needs comes as an argument, so that nothing is fetched through the kernel's parameter block
// byte after byte.
GTOK_DEV_NOINLINE uint32_t literal_in_window(const LitView lv, const uint8_t* win_txt, int lo, const uint8_t* text, const uint32_t* docmask,
                                             int s, int n, uint32_t* id_out) {
    auto byte_at = [&](int q) -> uint32_t {
        const int i = q - lo;
        return (i >= 0 && i < kPWin) ? win_txt[i] : ldg(text + q);
    };
    auto is_doc = [&](int q) -> bool { return q == 0 || (docmask && ((ldg(docmask + (q >> 5)) >> (q & 31)) & 1u)); };
    return match_literal_hashed(lv, docmask != nullptr, s, n, byte_at, is_doc, id_out);
}

// Class + flags of a byte, ignoring added tokens.  `byte_at(q)` must be valid for
// q in [p, p+3] when those are below n.
template <class GetByte, class IsDoc>
GTOK_DEV uint8_t plain_attr(const EncodeArgs& a, int p, int n, GetByte byte_at, IsDoc is_doc) {
    uint32_t b = byte_at(p);
    uint8_t flags = is_doc(p) ? A_DOC : 0;
    if ((b & 0xC0u) == 0x80u) return static_cast<uint8_t>(A_CONT | flags);
    uint32_t cp = b;
    if (b >= 0x80u) {
        // Lenient decode: the lead byte decides the width if that many bytes
        // remain in the document; continuation bytes are taken on trust.
        int avail = n - p;
        if (avail > 4) avail = 4;
        for (int k = 1; k < avail; ++k) if (is_doc(p + k)) { avail = k; break; }
        if ((b & 0xE0u) == 0xC0u && avail >= 2) cp = ((b & 0x1Fu) << 6) | (byte_at(p + 1) & 0x3Fu);
        else if ((b & 0xF0u) == 0xE0u && avail >= 3) cp = ((b & 0x0Fu) << 12) | ((byte_at(p + 1) & 0x3Fu) << 6) | (byte_at(p + 2) & 0x3Fu);
        else if ((b & 0xF8u) == 0xF0u && avail >= 4)
            cp = ((b & 0x07u) << 18) | ((byte_at(p + 1) & 0x3Fu) << 12) | ((byte_at(p + 2) & 0x3Fu) << 6) | (byte_at(p + 3) & 0x3Fu);
    }
    const bool wide = a.tb.uc_wide != 0;
    const uint32_t cls = uc_class([&](uint32_t i) { return static_cast<uint32_t>(ldg(a.tb.uc_stage1 + i)); }, [&](uint32_t i) { return ldg(a.tb.uc_stage2 + i); }, cp, wide);
    if (wide && cp_is_cjk(cp)) flags |= A_CJK;
    if (b == 0x0Au || b == 0x0Du) flags |= A_CRLF;
    if (b == 0x20u) flags |= A_SP;
    return static_cast<uint8_t>(cls | flags);
}

// Attribute of an arbitrary position straight from global memory (slow path for
// walks that leave the window).
GTOK_DEV_NOINLINE uint8_t attr_global(const EncodeArgs& a, int p, int n) {
    if (p < 0 || p >= n) return A_OUT;
    auto byte_at = [&](int q) -> uint32_t { return ldg(a.text + q); };
    auto is_doc = [&](int q) -> bool { return is_docstart_global(a, q); };
    bool may_be_in_literal = a.tb.added_max_bytes != 0;
    if (may_be_in_literal && a.tb.lit_first_n <= 4u) {
        // A literal that holds p starts at one of the few bytes a literal can start with, at most
        // added_max_bytes - 1 before p: the words that cover that stretch are fetched together and searched for
        // those byte values at once, so that the usual answer ("none there") costs one memory round trip.
        int lim = p - static_cast<int>(a.tb.added_max_bytes) + 1;
        if (lim < 0) lim = 0;
        const int w0 = lim >> 2, w1 = p >> 2;
        uint32_t found = 0;
        if (w1 - w0 < 16) {
            const uint32_t* tw = reinterpret_cast<const uint32_t*>(a.text);
            for (int wd = w0; wd <= w1; ++wd) {
                const uint32_t v = ldg(tw + wd);
                for (uint32_t f = 0; f < a.tb.lit_first_n; ++f) {
                    const uint32_t x = v ^ (((a.tb.lit_first >> (8 * f)) & 0xFFu) * 0x01010101u);
                    found |= (x - 0x01010101u) & ~x & 0x80808080u;          // some byte of the word may be that value
                }
            }
            if (!found) may_be_in_literal = false;
        }
    }
    if (may_be_in_literal) {
        // Only the nearest literal-start byte at or before p can own p: a literal
        // never contains another literal's first byte past its own first position.
        int lim = p - static_cast<int>(a.tb.added_max_bytes) + 1;
        if (lim < 0) lim = 0;
        for (int s = p; s >= lim; --s) {
            if (ldg(a.tb.trie_root + byte_at(s)) != kNoToken) {
                uint32_t id;
                uint32_t ml = longest_literal(a, s, n, byte_at, &id);
                if (ml && s + static_cast<int>(ml) > p) {
                    uint8_t flags = is_doc(p) ? A_DOC : 0;
                    return static_cast<uint8_t>((s == p ? A_ADDED : A_CONT) | flags);
                }
                break;
            }
            if (s < p && is_doc(s + 1)) break;   // never look into the previous document
        }
    }
    return plain_attr(a, p, n, byte_at, is_doc);
}

GTOK_DEV uint8_t attr_at(const Win& w, int p) {
    if (p >= w.vlo && p < w.vhi) return w.sm->attr[p - w.lo];
    return attr_global(*w.a, p, w.n);
}
GTOK_DEV uint32_t text_at(const Win& w, int p) {   // p in [0, n)
    if (p >= w.vlo && p < w.vhi) return w.sm->txt[p - w.lo];
    return ldg(w.a->text + p);
}

// Lead position of the codepoint before the one starting at p (p itself not a
// document start).  Returns -1 when p is the first codepoint of its document.
// (Outside the window a long stretch of stray continuation bytes is stepped over sixteen raw bytes at a
// time: a byte 10xxxxxx starts no codepoint whether or not an added-token literal holds it.)
GTOK_DEV bool no_docstart_in16(RawText t, int q);
GTOK_DEV bool sixteen_continuation_bytes(RawText t, int q) {      // q % 16 == 0; none opens a document
    if (!no_docstart_in16(t, q)) return false;
    const uint32_t* p4 = reinterpret_cast<const uint32_t*>(t.text + q);
    const uint32_t v0 = ldg(p4), v1 = ldg(p4 + 1), v2 = ldg(p4 + 2), v3 = ldg(p4 + 3);
    return ((v0 & v1 & v2 & v3) & 0x80808080u) == 0x80808080u && ((v0 | v1 | v2 | v3) & 0x40404040u) == 0u;
}
// The walks once they have left the window (q < w.vlo, q >= w.vhi): functions of their own, so that the
// many places that step from a codepoint to its neighbour carry only the look into shared memory.
GTOK_DEV_NOINLINE int prev_lead_far(const Win& w, int q) {
    const RawText t = raw_text(*w.a);
    for (;;) {
        if (q < 0) return -1;
        if ((q & 15) == 15 && q >= 31 && sixteen_continuation_bytes(t, q - 15)) { q -= 16; continue; }
        const uint8_t a = attr_global(*w.a, q, w.n);
        if ((a & A_CLS) != A_CONT) return q;
        if (a & A_DOC) return -1;
        --q;
    }
}
GTOK_DEV_NOINLINE int next_lead_far(const Win& w, int q) {
    const RawText t = raw_text(*w.a);
    const int n = w.n;
    for (;;) {
        if (q >= n) return -1;
        if ((q & 15) == 0 && q + 16 <= n && sixteen_continuation_bytes(t, q)) { q += 16; continue; }
        const uint8_t a = attr_global(*w.a, q, w.n);
        if (a & A_DOC) return -1;
        if ((a & A_CLS) != A_CONT) return q;
        ++q;
    }
}
GTOK_DEV int prev_lead(const Win& w, int p) {
    int q = p - 1;
    for (;;) {
        if (q < w.vlo || q >= w.vhi) return prev_lead_far(w, q);
        const uint8_t a = w.sm->attr[q - w.lo];
        if ((a & A_CLS) != A_CONT) return q;
        if (a & A_DOC) return -1;     // stray continuation bytes open the document: dropped
        --q;
    }
}
// Lead position of the codepoint after the one starting at p, or -1 at the end
// of the document.
GTOK_DEV int next_lead(const Win& w, int p) {
    int q = p + 1;
    for (;;) {
        if (q < w.vlo || q >= w.vhi) return next_lead_far(w, q);
        const uint8_t a = w.sm->attr[q - w.lo];
        if (a & A_DOC) return -1;
        if ((a & A_CLS) != A_CONT) return q;
        ++q;
    }
}
// Class of the codepoint at lead q for its neighbours: L/N/S/O, or -1 for "nothing
// there" (q < 0, or an added token, which behaves like the edge of the text).
GTOK_DEV int ncls(uint8_t a) {
    int c = a & A_CLS;
    return c <= A_O ? c : -1;
}

// Fast forms of the two run walks for positions outside the window, where every
// attribute would have to be rebuilt from global memory.  They only step over bytes
// whose meaning is certain from the byte alone (CR/LF going back, 0x20 going forward;
// never when an added-token literal could contain such a byte, never across a document
// start) and leave the deciding position to the general code.
// q is a CR/LF byte: position of the first byte before the newline stretch that is not
// CR/LF, or the CR/LF that opens its document (the caller's test then ends the walk).
GTOK_DEV bool all_bytes_in(uint32_t v, uint32_t x, uint32_t y) {   // every byte of v equals x or y
    for (int k = 0; k < 4; ++k) { uint32_t b = (v >> (8 * k)) & 0xFFu; if (b != x && b != y) return false; }
    return true;
}
GTOK_DEV bool no_docstart_in16(RawText t, int q) {    // q..q+15 within one mask word (q % 16 == 0)
    if (q == 0) return false;
    if (!t.docmask) return true;
    return ((ldg(t.docmask + (q >> 5)) >> (q & 31)) & 0xFFFFu) == 0;
}
GTOK_DEV bool no_docstart_in16(const EncodeArgs& a, int q) { return no_docstart_in16(raw_text(a), q); }
// True when the 128 bytes at q (q % 128 == 0) repeat one 4-byte pattern whose bytes are all x
// or y (CR/LF stretches: x = 0x0A, y = 0x0D; spaces: x = y = 0x20) and none of them opens a
// document.  The eight loads are independent and the test is two operations per word, so a long
// run is walked at about one memory round trip per 128 bytes.  (A stretch that mixes its two
// bytes irregularly is not recognised here and is walked 16 bytes at a time.)
GTOK_DEV bool run_of_128(RawText a, int q, uint32_t x, uint32_t y) {
    if (a.docmask) {
        const uint32_t* dm = a.docmask + (q >> 5);
        if (ldg(dm) | ldg(dm + 1) | ldg(dm + 2) | ldg(dm + 3)) return false;
    }
    uint32_t all_and = 0xFFFFFFFFu, all_or = 0;
#if defined(__CUDA_ARCH__)
    const uint4* p = reinterpret_cast<const uint4*>(a.text + q);
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = ld128(p + k);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        all_and &= v[k].x & v[k].y & v[k].z & v[k].w;
        all_or |= v[k].x | v[k].y | v[k].z | v[k].w;
    }
#else
    for (int k = 0; k < 32; ++k) {
        const uint8_t* t = a.text + q + 4 * k;
        const uint32_t w4 = static_cast<uint32_t>(t[0]) | (static_cast<uint32_t>(t[1]) << 8) | (static_cast<uint32_t>(t[2]) << 16) | (static_cast<uint32_t>(t[3]) << 24);
        all_and &= w4;
        all_or |= w4;
    }
#endif
    if (all_and != all_or) return false;               // the 32 words are not all the same
    return all_bytes_in(all_and, x, y);
}
// Inside the window, from the bit planes (16 bytes per entry, eight-byte aligned rows) and the window's
// document-start bits.  First window index in [i, i_end) whose byte is not a plain (non-newline) one-byte
// whitespace character of the running document, i_end when there is none: 64 bytes a step, 256 while whole
// groups of four are clean.  Pointers and bounds by value, in a function of its own: the loop then keeps
// everything in registers (a newline followed by a window full of spaces is 125 steps of 64, and one
// codepoint at a time through the attribute bytes costs a hundred times that).
GTOK_DEV int low_bit(uint64_t x) {
#if defined(__CUDA_ARCH__)
    return __ffsll(static_cast<long long>(x)) - 1;
#else
    return __builtin_ctzll(x);
#endif
}
GTOK_DEV int high_bit(uint64_t x) {
#if defined(__CUDA_ARCH__)
    return 63 - __clzll(static_cast<long long>(x));
#else
    return 63 - __builtin_clzll(x);
#endif
}
GTOK_DEV_NOINLINE int plain_ws_end(const uint16_t* ps, const uint16_t* pcr, const uint32_t* dsw, int i, int i_end) {
    if (i >= i_end) return i_end;
    const uint64_t* S = reinterpret_cast<const uint64_t*>(ps);
    const uint64_t* C = reinterpret_cast<const uint64_t*>(pcr);
    int g = i >> 6;
    uint64_t bad = (~S[g] | C[g] | dsw[2 * g] | (static_cast<uint64_t>(dsw[2 * g + 1]) << 32)) & (~0ull << (i & 63));
    for (;;) {
        if (bad) { const int j = g * 64 + low_bit(bad); return j < i_end ? j : i_end; }
        ++g;
        while (g * 64 + 256 <= i_end) {
            const uint64_t s_all = S[g] & S[g + 1] & S[g + 2] & S[g + 3], c_any = C[g] | C[g + 1] | C[g + 2] | C[g + 3];
            const uint32_t* d = dsw + 2 * g;
            const uint32_t d_any = d[0] | d[1] | d[2] | d[3] | d[4] | d[5] | d[6] | d[7];
            if (s_all != ~0ull || c_any != 0ull || d_any != 0u) break;
            g += 4;
        }
        if (g * 64 >= i_end) return i_end;
        bad = ~S[g] | C[g] | dsw[2 * g] | (static_cast<uint64_t>(dsw[2 * g + 1]) << 32);
    }
}
// The same going back over newline bytes: the lowest window index j in [i_begin, i] such that j..i are all
// newline bytes none of which opens a document (i + 1 when the byte at i is not such a one).
GTOK_DEV_NOINLINE int newline_run_begin(const uint16_t* pcr, const uint32_t* dsw, int i, int i_begin) {
    if (i < i_begin) return i + 1;
    const uint64_t* C = reinterpret_cast<const uint64_t*>(pcr);
    int g = i >> 6;
    uint64_t bad = (~C[g] | dsw[2 * g] | (static_cast<uint64_t>(dsw[2 * g + 1]) << 32)) & (~0ull >> (63 - (i & 63)));
    for (;;) {
        if (bad) { const int j = g * 64 + high_bit(bad) + 1; return j > i_begin ? j : i_begin; }
        if (g * 64 <= i_begin) return i_begin;
        --g;
        bad = ~C[g] | dsw[2 * g] | (static_cast<uint64_t>(dsw[2 * g + 1]) << 32);
    }
}
GTOK_DEV int skip_back_newlines(const Win& w, int q) {
    if (w.a->tb.added_ws) return q;
    const RawText a = raw_text(*w.a);
    const int far = w.sm->far_run[2];              // from here on the whole block has looked already (far_runs); -2: nowhere
    for (;;) {
        if (q < 0) return q;
        if (q == far) return w.sm->far_run[3];
        const bool over128 = q > far && q - 128 < far, over16 = q > far && q - 16 < far;      // never step over that place
        if ((q & 127) == 127 && q >= 255 && !over128 && run_of_128(a, q - 127, 0x0Au, 0x0Du)) { q -= 128; continue; }
        if ((q & 15) == 15 && q >= 31 && !over16 && no_docstart_in16(a, q - 15)) {
            const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + q - 15);
            uint32_t v0 = ldg(p4), v1 = ldg(p4 + 1), v2 = ldg(p4 + 2), v3 = ldg(p4 + 3);
            if (all_bytes_in(v0, 0x0Au, 0x0Du) && all_bytes_in(v1, 0x0Au, 0x0Du) && all_bytes_in(v2, 0x0Au, 0x0Du) && all_bytes_in(v3, 0x0Au, 0x0Du)) { q -= 16; continue; }
        }
        uint32_t b = ldg(a.text + q);
        if (b != 0x0Au && b != 0x0Du) return q;
        if (raw_docstart(a, q)) return q;
        --q;
    }
}
// r is a lead at or past the window end: first position at or after r that is not the byte `sp` (a
// plain space, or another one-byte ASCII whitespace character) of the same document, or -1 at the
// end of the document.
GTOK_DEV int skip_forward_spaces(const Win& w, int r, uint32_t sp = 0x20u) {
    if (w.a->tb.added_ws) return r;
    const RawText a = raw_text(*w.a);
    const int n = w.n;
    const uint32_t sp4 = sp * 0x01010101u;
    const int far = w.sm->far_run[0];              // from here on the whole block has looked already (far_runs); -2: nowhere
    for (;;) {
        if (r >= n) return -1;
        if (r == far) return w.sm->far_run[1];
        const bool over128 = r < far && r + 128 > far, over16 = r < far && r + 16 > far;          // never step over that place
        if ((r & 127) == 0 && r > 0 && r + 128 <= n && !over128 && run_of_128(a, r, sp, sp)) { r += 128; continue; }
        if ((r & 15) == 0 && r + 16 <= n && !over16 && no_docstart_in16(a, r)) {
            const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + r);
            if (ldg(p4) == sp4 && ldg(p4 + 1) == sp4 && ldg(p4 + 2) == sp4 && ldg(p4 + 3) == sp4) { r += 16; continue; }
        }
        if (raw_docstart(a, r)) return -1;
        if (ldg(a.text + r) != sp) return r;
        ++r;
    }
}
// r is the lead of a two- or three-byte codepoint that is not part of an added-token literal: first position
// after the stretch in which that same codepoint is repeated within the document (r itself when it is not
// repeated, or when its bytes could open a literal).  Raw bytes only: a literal cannot begin inside such a
// stretch when none of the codepoint's bytes is the first byte of a literal, and one that began before it
// would hold r too.  (A no-break space or an ideographic space repeated for kilobytes after a newline is
// walked this way instead of one attribute at a time.)
GTOK_DEV_NOINLINE int skip_forward_repeat(const Win& w, int r) {
    const EncodeArgs& args = *w.a;
    const RawText a = raw_text(args);
    const int n = w.n;
    const uint32_t b0 = ldg(a.text + r);
    const int width = b0 >= 0xE0u ? 3 : 2;
    if (b0 < 0xC2u || b0 >= 0xF0u || r + width > n) return r;
    const uint32_t b1 = ldg(a.text + r + 1), b2 = width == 3 ? ldg(a.text + r + 2) : 0u;
    if ((b1 & 0xC0u) != 0x80u || (width == 3 && (b2 & 0xC0u) != 0x80u)) return r;
    if (((args.tb.lit1_bits[b0 >> 5] >> (b0 & 31)) | (args.tb.lit1_bits[b1 >> 5] >> (b1 & 31)) | (width == 3 ? args.tb.lit1_bits[b2 >> 5] >> (b2 & 31) : 0u)) & 1u) return r;
    for (int k = 1; k < width; ++k) if (raw_docstart(a, r + k)) return r;
    int q = r + width;
    for (;;) {
        if (q + width > n) return q;
        if (ldg(a.text + q) != b0 || ldg(a.text + q + 1) != b1 || (width == 3 && ldg(a.text + q + 2) != b2)) return q;
        for (int k = 0; k < width; ++k) if (raw_docstart(a, q + k)) return q;
        q += width;
    }
}
// r is the lead of a whitespace codepoint: where to go on from when that codepoint is repeated (the last
// of the repeats, so that the caller looks at it and steps on as usual), r itself when it is not, -1 when
// the repeats run to the end of the document.
GTOK_DEV_NOINLINE int skip_forward_ws_run(const Win& w, int r) {
    const uint32_t sp = text_at(w, r);
    if (sp == 0x20u || sp == 0x09u || sp == 0x0Bu || sp == 0x0Cu) {
        const int e = sp == 0x20u ? skip_forward_spaces(w, r, 0x20u) : skip_forward_spaces(w, r, sp);     // (the usual byte as a constant)
        return e < 0 ? -1 : (e > r ? e - 1 : r);
    }
    if (sp >= 0xC2u) {
        const uint8_t a_r = attr_at(w, r);
        if ((a_r & A_CLS) == A_S && !(a_r & A_CRLF)) { const int e = skip_forward_repeat(w, r); if (e > r) return e - (sp >= 0xE0u ? 3 : 2); }
    }
    return r;
}
// q is an ASCII letter outside any added-token literal: position of the first byte before the run of
// ASCII letters it stands in that is not one, or the letter that opens its document.  Whole words of
// four letters are stepped over sixteen bytes at a time (a literal's bytes would read as letters too:
// the caller asks only when no literal ends with a letter, so that a literal always shows its last,
// other byte first).
GTOK_DEV bool four_letters(uint32_t v) {
    const uint32_t lo7 = (v | 0x20202020u) & 0x7F7F7F7Fu;
    const uint32_t ge_a = lo7 + (0x80u - 'a') * 0x01010101u, gt_z = lo7 + (0x80u - 'z' - 1u) * 0x01010101u;
    return (ge_a & ~gt_z & ~v & 0x80808080u) == 0x80808080u;
}
// True when the 128 bytes at q (q % 128 == 0) are all ASCII letters and none of them opens a document
// (eight independent loads, as in run_of_128).
GTOK_DEV bool letters_128(RawText a, int q) {
    if (a.docmask) {
        const uint32_t* dm = a.docmask + (q >> 5);
        if (ldg(dm) | ldg(dm + 1) | ldg(dm + 2) | ldg(dm + 3)) return false;
    }
    bool ok = true;
#if defined(__CUDA_ARCH__)
    const uint4* p = reinterpret_cast<const uint4*>(a.text + q);
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = ld128(p + k);
#pragma unroll
    for (int k = 0; k < 8; ++k) ok = ok && four_letters(v[k].x) && four_letters(v[k].y) && four_letters(v[k].z) && four_letters(v[k].w);
#else
    for (int k = 0; k < 32; ++k) {
        const uint8_t* t = a.text + q + 4 * k;
        ok = ok && four_letters(static_cast<uint32_t>(t[0]) | (static_cast<uint32_t>(t[1]) << 8) | (static_cast<uint32_t>(t[2]) << 16) | (static_cast<uint32_t>(t[3]) << 24));
    }
#endif
    return ok;
}
GTOK_DEV int skip_back_letters(const Win& w, int q) {
    const RawText a = raw_text(*w.a);
    for (;;) {
        if (q < 0) return q;
        if ((q & 127) == 127 && q >= 255 && letters_128(a, q - 127)) { q -= 128; continue; }
        if ((q & 15) == 15 && q >= 31 && no_docstart_in16(a, q - 15)) {
            const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + q - 15);
            const uint32_t v0 = ldg(p4), v1 = ldg(p4 + 1), v2 = ldg(p4 + 2), v3 = ldg(p4 + 3);
            if (four_letters(v0) && four_letters(v1) && four_letters(v2) && four_letters(v3)) { q -= 16; continue; }
        }
        const uint32_t b = ldg(a.text + q);
        if (!((b >= 'a' && b <= 'z') || (b >= 'A' && b <= 'Z'))) return q;
        if (raw_docstart(a, q)) return q;
        --q;
    }
}

// First byte of the codepoint at lead q as the contraction rule sees it:
// lower-cased ASCII and U+017F read as 's' when the family matches case-insensitively.
GTOK_DEV int tail_byte(const Win& w, int q, bool ci) {
    if (q < 0) return -1;
    uint8_t a = attr_at(w, q);
    if ((a & A_CLS) > A_O) return -1;
    int b = static_cast<int>(text_at(w, q));
    if (ci) {
        if (b >= 'A' && b <= 'Z') b += 32;
        else if (b == 0xC5 && q + 1 < w.n && !(attr_at(w, q + 1) & A_DOC) && text_at(w, q + 1) == 0xBF) b = 's';
    }
    return b;
}

// Does a contraction ('s 't 'm 'd -> 1, 're 've 'll -> 2) start at the apostrophe
// at lead k?  It does when the letters follow and the regex cursor can be at k:
// at the start of the document, or after anything but punctuation or a literal space.
GTOK_DEV int contraction_at(const Win& w, int k, uint8_t ak, bool ci) {
    if ((ak & A_CLS) != A_O || text_at(w, k) != 0x27u) return 0;
    int r1 = next_lead(w, k);
    if (r1 < 0) return 0;
    int x = tail_byte(w, r1, ci), tl = 0;
    if (x == 'r' || x == 'v' || x == 'l') {
        int r2 = next_lead(w, r1);
        int y = r2 < 0 ? -1 : tail_byte(w, r2, ci);
        if ((x == 'l' && y == 'l') || (x != 'l' && y == 'e')) tl = 2;
    } else if (x == 's' || x == 't' || x == 'm' || x == 'd') tl = 1;
    if (!tl) return 0;
    if (ak & A_DOC) return tl;
    int q = prev_lead(w, k);
    if (q < 0) return tl;
    uint8_t aq = attr_at(w, q);
    if ((aq & A_CLS) == A_O) return 0;
    if ((aq & A_CLS) == A_S && (aq & A_SP)) return 0;
    return tl;
}
GTOK_DEV int contraction_at(const Win& w, int k, bool ci) {
    if (k < 0) return 0;
    return contraction_at(w, k, attr_at(w, k), ci);
}

// ---- DeepSeek-V3 ----
// Three Split steps one after the other (src/vocab.cc:132-137 of the reference): numbers in
// threes, runs inside the three CJK ranges, then the main pattern on every piece the first two
// left, for which a piece's ends are the ends of the text.  Where the main pattern's matches
// start follows from the codepoints next to a position (the alternatives are tried in order at
// each place, but which one wins is settled by what a place and its neighbours are), with three
// walks: back along ASCII letters to the punctuation mark that may have taken them along, back
// over newlines to the punctuation whose match swallowed them, forward over whitespace to a later
// newline.  Classes here: A_L letters and marks, A_N, A_S whitespace, A_P punctuation and symbols,
// A_O the rest (matched by nothing unless a letter follows).
GTOK_DEV int dcls(uint8_t a) {            // class of a neighbour, -1 for "nothing there" (an added token, outside)
    const int c = a & A_CLS;
    return (c <= A_O || c == A_P) ? c : -1;
}
GTOK_DEV bool ascii_letter(uint32_t b) { return (b >= 'a' && b <= 'z') || (b >= 'A' && b <= 'Z'); }
GTOK_DEV bool ascii_punct(uint32_t b) { return (b >= 0x21u && b <= 0x2Fu) || (b >= 0x3Au && b <= 0x40u) || (b >= 0x5Bu && b <= 0x60u) || (b >= 0x7Bu && b <= 0x7Eu); }
// Do the codepoints with attributes x and y (neither an added token nor outside) lie in one piece of
// the first two steps?  Numbers are pieces of their own, and a piece is inside or outside the CJK ranges.
GTOK_DEV bool ds_same_piece(uint8_t x, uint8_t y) {
    if ((x & A_CLS) == A_N || (y & A_CLS) == A_N) return false;
    return ((x ^ y) & A_CJK) == 0;
}
// Lead of the codepoint before / after the one at p (attribute ap) inside p's piece, or -1.
GTOK_DEV int ds_prev(const Win& w, int p, uint8_t ap, uint8_t* aq) {
    if (ap & A_DOC) return -1;
    const int q = prev_lead(w, p);
    if (q < 0) return -1;
    *aq = attr_at(w, q);
    if (dcls(*aq) < 0 || !ds_same_piece(*aq, ap)) return -1;
    return q;
}
GTOK_DEV int ds_next(const Win& w, int p, uint8_t ap, uint8_t* ar) {
    const int r = next_lead(w, p);
    if (r < 0) return -1;
    *ar = attr_at(w, r);
    if (dcls(*ar) < 0 || !ds_same_piece(*ar, ap)) return -1;
    return r;
}
// Does the first alternative (one ASCII punctuation mark, then ASCII letters) start a match at the
// mark at m?  It does when a letter follows and the scan can be at m: the mark is not inside a run
// of punctuation and not behind the space such a run takes along.
GTOK_DEV bool ds_mark_takes_letters(const Win& w, int m, uint8_t am) {
    if (!ascii_punct(text_at(w, m))) return false;
    uint8_t ar, aq;
    const int r = ds_next(w, m, am, &ar);
    if (r < 0 || !ascii_letter(text_at(w, r))) return false;
    const int q = ds_prev(w, m, am, &aq);
    if (q < 0) return true;
    return !((aq & A_CLS) == A_P || (aq & A_SP));
}
// ---- Gemma-3 shape ----
// The model merges the characters of the whole text, so any cut must be one that no rule can reach across.  Two
// kinds are taken.  A byte that is not part of a whole character of the vocabulary (a character the vocabulary lacks,
// malformed UTF-8, a character cut by a document's end) stands alone: the model spells it as its "<0xNN>" token,
// which no rule mentions, and keeping such bytes apart is also what keeps the loader's byte-to-character rules from
// ever seeing them.  And a space (U+0020, which the normaliser writes as U+2581, or that character itself) opens a
// pre-token unless some rule's left side ends with the character before it while its right side begins with U+2581
// (class 6 in the vocabulary's class table; 0 any other character of the vocabulary, 3 everything else).
// Every byte of the tile is decided here, by strict decoding of the bytes around it.
GTOK_DEV bool sp_docstart_at(const Win& w, int p) {
    const int i = p - w.lo;
    if (i >= 0 && i < kPWin) return (w.sm->dsw[i >> 5] >> (i & 31)) & 1u;
    return is_docstart_global(*w.a, p);
}
// The whole character that holds byte p, inside p's document: its first byte in *start, its codepoint in *cp; 0 when
// there is none, else its width.
GTOK_DEV int sp_char_at(const Win& w, int p, int* start, uint32_t* cp) {
    int s = p;
    for (int k = 0; (text_at(w, s) & 0xC0u) == 0x80u; ++k) {
        if (k == 3 || s == 0 || sp_docstart_at(w, s)) return 0;
        --s;
    }
    const uint32_t b0 = text_at(w, s);
    int width;
    if (b0 < 0x80u) width = 1;
    else if (b0 >= 0xC2u && b0 <= 0xDFu) width = 2;
    else if (b0 >= 0xE0u && b0 <= 0xEFu) width = 3;
    else if (b0 >= 0xF0u && b0 <= 0xF4u) width = 4;
    else return 0;
    if (s + width > w.n || p >= s + width) return 0;
    uint32_t v = width == 1 ? b0 : width == 2 ? (b0 & 0x1Fu) : width == 3 ? (b0 & 0x0Fu) : (b0 & 0x07u);
    for (int k = 1; k < width; ++k) {
        const uint32_t b = text_at(w, s + k);
        if ((b & 0xC0u) != 0x80u || sp_docstart_at(w, s + k)) return 0;
        v = (v << 6) | (b & 0x3Fu);
    }
    if ((width == 3 && (v < 0x800u || (v >= 0xD800u && v <= 0xDFFFu))) || (width == 4 && (v < 0x10000u || v > 0x10FFFFu))) return 0;
    *start = s;
    *cp = v;
    return width;
}
// Class of the whole character cp that begins at s.  Inside the window the classification phase has looked it up already
// (a well-formed sequence decodes there to the same codepoint); outside, from the table in global memory.
GTOK_DEV uint32_t sp_class(const Win& w, int s, uint32_t cp) {
    if (s >= w.vlo && s < w.vhi) {
        const uint32_t k = w.sm->attr[s - w.lo] & A_CLS;
        if (k == 0u || k == 3u || k == 6u) return k;              // (an added token's bytes carry another class: the long way then)
    }
    const EncodeArgs& a = *w.a;
    return uc_class([&](uint32_t i) { return static_cast<uint32_t>(ldg(a.tb.uc_stage1 + i)); }, [&](uint32_t i) { return ldg(a.tb.uc_stage2 + i); }, cp, true);
}
GTOK_DEV_NOINLINE bool is_boundary_sp(const Win& w, int p) {
    if (p == 0 || sp_docstart_at(w, p)) return true;
    int s = 0, s1 = 0;
    uint32_t cp = 0, c1 = 0;
    if (!sp_char_at(w, p, &s, &cp) || sp_class(w, s, cp) == 3u) return true;       // on its own, byte by byte
    if (s != p) return false;                                                         // inside a character
    // what ends right before p: an added token, a byte on its own, or a character
    const int q = prev_lead(w, p);
    if (q < 0 || (attr_at(w, q) & A_CLS) == A_ADDED) return true;
    if (!sp_char_at(w, p - 1, &s1, &c1)) return true;
    const uint32_t k1 = sp_class(w, s1, c1);
    if (k1 == 3u) return true;
    if (cp == 0x20u || cp == 0x2581u) return k1 != 6u;
    return false;
}

GTOK_DEV_NOINLINE bool is_boundary_deepseek(const Win& w, int p, uint8_t a0, bool* pending, bool* nstart) {
    *pending = false;
    const int cur = a0 & A_CLS;
    if (cur == A_N) *nstart = true;
    if (a0 & A_DOC) return true;
    const int q = prev_lead(w, p);
    if (q < 0) return true;
    const uint8_t a1 = attr_at(w, q);
    const int prev = dcls(a1);
    if (prev < 0) return true;                               // after an added token
    if (cur == A_N) {
        if (prev != A_N) return true;
        *nstart = false;
        *pending = true;                                     // its place in the run decides (every third one starts a piece)
        return false;
    }
    if (!ds_same_piece(a1, a0)) return true;                 // after a number, or into / out of the CJK ranges
    const bool pcrlf = (a1 & A_CRLF) != 0;
    if (cur == A_L) {
        if (prev == A_L) {
            // inside a run of letters: only where ASCII letters that a punctuation mark took along end
            if (!ascii_letter(text_at(w, q)) || ascii_letter(text_at(w, p))) return false;
            int k = q;
            uint8_t ak = a1;
            for (;;) {
                if (k > 0 && !w.a->tb.added_alpha_end && !(ak & A_DOC) && ascii_letter(text_at(w, k - 1))) {
                    // over raw bytes, sixteen at a time (one codepoint at a time a long run would hold its tile up)
                    const int r = skip_back_letters(w, k - 1);
                    if (r < k - 1) {
                        const uint32_t br = r >= 0 ? text_at(w, r) : 0u;
                        k = (r >= 0 && ascii_letter(br)) ? r : r + 1;        // a letter there opens its document
                        ak = attr_at(w, k);
                    }
                }
                uint8_t aj;
                const int j = ds_prev(w, k, ak, &aj);
                if (j < 0) return false;
                if ((aj & A_CLS) == A_L && ascii_letter(text_at(w, j))) { k = j; ak = aj; continue; }
                return ds_mark_takes_letters(w, j, aj);
            }
        }
        if (prev == A_S) return pcrlf;                       // one whitespace codepoint (no newline) or one "other" leads the letters
        if (prev == A_O) return false;
        // prev == A_P
        return !(ascii_letter(text_at(w, p)) && ds_mark_takes_letters(w, q, a1));
    }
    if (cur == A_P) return !(prev == A_P || (a1 & A_SP));
    if (cur == A_S && (a0 & A_CRLF)) return prev == A_L || prev == A_O;     // else behind punctuation (taken along) or inside whitespace
    if (cur == A_S) {
        if (prev != A_S) return true;
        if (pcrlf) {
            // newlines before: taken along by punctuation (then whitespace starts afresh here), or part of
            // a whitespace match that runs on through its last newline
            int k = q;
            uint8_t ak = a1;
            for (;;) {
                if (k - 1 >= w.vlo && k - 1 < w.vhi && !(ak & A_DOC)) {
                    // inside the window: down to the first of the newline bytes that end before k, from the bit planes
                    const int i2 = newline_run_begin(w.sm->plane[PL_CRLF], w.sm->dsw, k - 1 - w.lo, w.vlo - w.lo);
                    if (w.lo + i2 < k - 1) { k = w.lo + i2; ak = attr_at(w, k); }
                }
                if (k > 0 && !(ak & A_DOC) && (text_at(w, k - 1) == 0x0Au || text_at(w, k - 1) == 0x0Du)) {
                    // over raw bytes, up to 128 at a time
                    const int r = skip_back_newlines(w, k - 1);
                    if (r < k - 1) {
                        const uint32_t br = r >= 0 ? text_at(w, r) : 0u;
                        k = (r >= 0 && (br == 0x0Au || br == 0x0Du)) ? r : r + 1;        // a newline there opens its document
                        ak = attr_at(w, k);
                    }
                }
                uint8_t aj;
                const int j = ds_prev(w, k, ak, &aj);
                if (j < 0) break;
                if (aj & A_CRLF) { k = j; ak = aj; continue; }
                if ((aj & A_CLS) == A_P) return true;
                break;
            }
            k = p;
            ak = a0;
            for (;;) {
                if (k + 1 >= w.vlo && k + 1 < w.vhi) {
                    // inside the window: on to the last byte before the first one that is not plain one-byte whitespace, from the bit planes
                    const int j = plain_ws_end(w.sm->plane[PL_S], w.sm->plane[PL_CRLF], w.sm->dsw, k + 1 - w.lo, w.vhi - w.lo);
                    if (w.lo + j - 1 > k) { k = w.lo + j - 1; ak = attr_at(w, k); }
                }
                {
                    // the same whitespace codepoint again and again: over raw bytes
                    const int e = skip_forward_ws_run(w, k);
                    if (e < 0) return true;                           // whitespace to the end of the document
                    if (e > k) { k = e; ak = attr_at(w, k); }
                }
                uint8_t aj;
                const int j = ds_next(w, k, ak, &aj);
                if (j < 0 || (aj & A_CLS) != A_S) return true;
                if (aj & A_CRLF) return false;
                k = j; ak = aj;
            }
        }
        // inside plain whitespace: the last codepoint before a non-space stays behind for what follows
        uint8_t ar;
        const int r = ds_next(w, p, a0, &ar);
        return r >= 0 && (ar & A_CLS) != A_S;
    }
    // cur == A_O
    if (prev != A_O) return true;
    uint8_t ar;
    const int r = ds_next(w, p, a0, &ar);
    return r >= 0 && (ar & A_CLS) == A_L;
}

// Boundary decision for the lead byte at p with attribute a0 (class L/N/S/O).
// Sets *pending for a Llama-3 digit inside a digit run, whose answer depends on
// its index in the run and is filled in later.
GTOK_DEV bool is_boundary(const Win& w, int p, uint8_t a0, uint32_t family, bool* pending, bool* nstart) {
    *pending = false;
    const int cur = a0 & A_CLS;
    const bool ci = family != 0;
    int q1 = (a0 & A_DOC) ? -1 : prev_lead(w, p);
    if (cur == A_N) *nstart = true;
    if (q1 < 0) return true;                       // first codepoint of its document
    const uint8_t a1 = attr_at(w, q1);
    const int prev = ncls(a1);
    if (cur == A_N && prev == A_N) *nstart = false;

    if (cur == A_L) {
        // Inside a contraction tail?
        int c1 = contraction_at(w, q1, a1, ci);
        if (c1 >= 1) return false;
        if (prev == A_L) {
            int q2 = (a1 & A_DOC) ? -1 : prev_lead(w, q1);
            if (q2 >= 0) {
                int c2 = contraction_at(w, q2, ci);
                if (c2 == 2) return false;          // second letter of 're 've 'll
                if (c2 == 1) return true;           // letter right after a finished 's 't 'm 'd
                uint8_t a2 = attr_at(w, q2);
                int q3 = (a2 & A_DOC) ? -1 : prev_lead(w, q2);
                if (q3 >= 0 && contraction_at(w, q3, ci) == 2) return true;   // after a finished 're 've 'll
            }
            return false;                            // inside a run of letters
        }
    } else if (cur == A_O) {
        if (contraction_at(w, p, a0, ci)) return true;
    }

    if (family == 0) {   // ---------------------------------------------- GPT-2
        if (prev == A_S && (a1 & A_SP) && cur != A_S) return false;      // " x": the space leads the token
        if (cur == A_S) {
            if (prev != A_S) return true;
            // Last whitespace before a non-space splits off (\s+(?!\S)).
            int r1 = next_lead(w, p);
            if (r1 < 0) return false;
            int nx = ncls(attr_at(w, r1));
            return nx >= 0 && nx != A_S;
        }
        return cur != prev;
    }

    // ----------------------------------------------------------- Llama-3 / Qwen2.5
    if (cur == A_S) {
        if (a0 & A_CRLF) return prev == A_L || prev == A_N || prev < 0;   // else absorbed (O) or inside a run (S)
        if (prev != A_S) return true;                                     // the run starts here
        if (!(a1 & A_CRLF)) {
            // Plain whitespace after plain whitespace: only the run's last char,
            // with something other than the end of the text after it, splits off.
            int r1 = next_lead(w, p);
            if (r1 < 0) return false;
            int nx = ncls(attr_at(w, r1));
            return nx >= 0 && nx != A_S;
        }
        // Previous char is CR/LF.  If that newline stretch hangs off a punctuation
        // token ( ?[^\s\p{L}\p{N}]+[\r\n]*), the whitespace run starts here.
        int q = q1;
        for (;;) {
            if (q < w.vlo) q = skip_back_newlines(w, q);      // long runs: raw bytes, 128 or 16 at a time
            if (q < 0) break;
            if (q >= w.vlo && q < w.vhi) {
                // inside the window: down to the first of the newline bytes that end at q, from the bit planes
                const int i2 = newline_run_begin(w.sm->plane[PL_CRLF], w.sm->dsw, q - w.lo, w.vlo - w.lo);
                if (w.lo + i2 < q) q = w.lo + i2;
            }
            uint8_t aq = attr_at(w, q);
            if (!((aq & A_CLS) == A_S && (aq & A_CRLF))) { if ((aq & A_CLS) == A_O) return true; break; }
            if (aq & A_DOC) break;
            q = prev_lead(w, q);
            if (q < 0) break;
        }
        // Otherwise p follows a newline inside the run: it starts the remainder
        // only if no later newline in the run pulls it into \s*[\r\n]+.
        int r = p;
        for (;;) {
            if (r + 1 >= w.vlo && r + 1 < w.vhi) {
                // inside the window: on to the last byte before the first one that is not plain one-byte whitespace, from the bit planes
                const int j = plain_ws_end(w.sm->plane[PL_S], w.sm->plane[PL_CRLF], w.sm->dsw, r + 1 - w.lo, w.vhi - w.lo);
                if (w.lo + j - 1 > r) r = w.lo + j - 1;
            }
            r = next_lead(w, r);
            if (r < 0) return true;
            if (r >= w.vhi) {
                const int r2 = skip_forward_ws_run(w, r);
                if (r2 < 0) return true;
                if (r2 > r) {
                    // r2 is the last of the repeats (plain whitespace, as r is).  The usual byte after it settles the
                    // question without classifying anything: an ASCII newline, or ASCII that is no whitespace.
                    r = r2;
                    if (r + 1 < w.n) {
                        const uint32_t b = ldg(w.a->text + r + 1);
                        const bool other_doc = is_docstart_global(*w.a, r + 1);
                        if (!other_doc && (b == 0x0Au || b == 0x0Du)) return false;
                        if (other_doc || (b > 0x20u && b < 0x80u)) return true;
                    }
                    continue;
                }
            }
            uint8_t ar = attr_at(w, r);
            if ((ar & A_CLS) != A_S) return true;
            if (ar & A_CRLF) return false;
        }
    }
    if (cur == A_L) {
        if (prev == A_S) return (a1 & A_CRLF) != 0;     // any non-newline whitespace leads the word
        if (prev == A_O) {
            // One punctuation char leads the word if the cursor can be at it.
            if (a1 & A_DOC) return false;
            int q2 = prev_lead(w, q1);
            if (q2 < 0) return false;
            uint8_t a2 = attr_at(w, q2);
            if ((a2 & A_CLS) == A_O) return true;
            if ((a2 & A_CLS) == A_S && (a2 & A_SP)) return true;
            return false;
        }
        return true;
    }
    if (cur == A_N) {
        if (family == 2 || prev != A_N) return true;
        *pending = true;
        return false;
    }
    // cur == A_O
    if (prev == A_O) return false;
    if (prev == A_S && (a1 & A_SP)) return false;
    return true;
}

// Once per block, before its first tile: the byte table and the block's copy of the class table.
// kWide: the vocabulary is of the DeepSeek-V3 family (wide class table, its own boundary rules); a
// template parameter so that the other families' kernel carries none of that code.
template <bool kWide, class Blk>
GTOK_DEV void pretok_block_init(Blk& blk, const EncodeArgs& a, PretokSmem& sm) {
    blk.par([&](int tid) {
        constexpr bool wide = kWide;              // the wide table is larger than the block's copy: it stays in global memory
        if (!wide) {
#if defined(__CUDA_ARCH__)
            // 128-bit copies (both arrays are whole multiples of 16 bytes and 16-byte aligned in device memory)
            for (int i = tid; i < kUcStage1Bmp / 8; i += kThreads) reinterpret_cast<uint4*>(sm.ucs1)[i] = __ldg(reinterpret_cast<const uint4*>(a.tb.uc_stage1) + i);
            for (int i = tid; i < kUcStage2Words / 4; i += kThreads) reinterpret_cast<uint4*>(sm.ucs2)[i] = __ldg(reinterpret_cast<const uint4*>(a.tb.uc_stage2) + i);
#else
            for (int i = tid; i < kUcStage1Bmp; i += kThreads) sm.ucs1[i] = ldg(a.tb.uc_stage1 + i);
            for (int i = tid; i < kUcStage2Words; i += kThreads) sm.ucs2[i] = ldg(a.tb.uc_stage2 + i);
#endif
        }
        uint8_t at;
        if (tid < 128) {
            at = static_cast<uint8_t>(uc_class([&](uint32_t i) { return static_cast<uint32_t>(ldg(a.tb.uc_stage1 + i)); },
                                               [&](uint32_t i) { return ldg(a.tb.uc_stage2 + i); }, static_cast<uint32_t>(tid), wide));
            if (tid == 0x0A || tid == 0x0D) at |= A_CRLF;
            if (tid == 0x20) at |= A_SP;
        } else at = tid < 0xC0 ? A_CONT : A_O;
        if (tid < kLitLens) sm.lit_lens[tid] = a.tb.lit_lens[tid];
        sm.lut[tid] = at | (static_cast<uint32_t>(onehot_of(at)) << 8) | (((a.tb.lit1_bits[tid >> 5] >> (tid & 31)) & 1u) << 16);
    });
}

// Runs that leave the tile's window, found by the whole block.  A walk along a run of newlines or of one
// whitespace byte is one thread's work, 128 bytes a step, while the rest of the block waits: a 36 KB run of
// spaces after a newline is 280 steps, longer than everything else the tile does.  So before the rules are
// applied, when the window ends inside a run of one ASCII whitespace byte, all threads look for that run's
// end together, 4 KB a step; likewise backwards from the window's start inside a stretch of newlines.  The
// walks (skip_forward_ws_run, skip_back_newlines) take the answer when they arrive at the window's edge.
template <class Blk>
GTOK_DEV void far_runs(Blk& blk, const EncodeArgs& a, PretokSmem& sm, int lo, int vlo, int vhi, int n) {
    blk.par([&](int tid) {
        if (tid != 0) return;
        if (vhi < n && vhi - 1 >= vlo) {
            const uint32_t sp = sm.txt[vhi - 1 - lo];
            if ((sp == 0x20u || sp == 0x09u || sp == 0x0Bu || sp == 0x0Cu) && ldg(a.text + vhi) == sp && !is_docstart_global(a, vhi)) sm.far_run[0] = vhi;
        }
        if (vlo >= 2 && vlo < vhi) {
            const uint32_t b0 = sm.txt[vlo - lo], b1 = ldg(a.text + vlo - 1);
            if ((b0 == 0x0Au || b0 == 0x0Du) && (b1 == 0x0Au || b1 == 0x0Du) && !is_docstart_global(a, vlo)) sm.far_run[2] = vlo - 1;
        }
    });
    if (sm.far_run[0] >= 0) {
        // what skip_forward_spaces(vhi) returns: the first position that is not that byte, or -1 when the document ends first
        const uint32_t sp = sm.txt[vhi - 1 - lo];
        int answer = -1;
        for (int base = vhi;; base += 64 * kThreads) {
            blk.par([&](int tid) {
                // sixty-four bytes a thread, sixteen at a time (the window's end is a multiple of 16)
                uint32_t first = 0xFFFFFFFFu;
                const uint32_t sp4 = sp * 0x01010101u;
                for (int c = 0; c < 4 && first == 0xFFFFFFFFu; ++c) {
                    const int q0 = base + 64 * tid + 16 * c;
                    if (q0 + 16 <= n && no_docstart_in16(a, q0)) {
                        const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + q0);
                        if (ldg(p4) == sp4 && ldg(p4 + 1) == sp4 && ldg(p4 + 2) == sp4 && ldg(p4 + 3) == sp4) continue;
                    }
                    for (int k = 0; k < 16 && first == 0xFFFFFFFFu; ++k) {
                        const int q = q0 + k;
                        if (q >= n || is_docstart_global(a, q) || ldg(a.text + q) != sp) first = static_cast<uint32_t>(q);
                    }
                }
                sm.scan[tid] = first;
            });
            const uint32_t m = blk.reduce_min(sm.scan);
            if (m != 0xFFFFFFFFu) {
                const int q = static_cast<int>(m);
                answer = (q >= n || is_docstart_global(a, q)) ? -1 : q;
                break;
            }
        }
        blk.par([&](int tid) { if (tid == 0) sm.far_run[1] = answer; });
    }
    if (sm.far_run[2] >= 0) {
        // what skip_back_newlines(vlo - 1) returns: the first position going back that holds no newline byte, or a
        // newline that opens its document, or -1
        int answer = -1;
        // (the bytes from the last 16-byte line below the window's start up to that start first, by one thread's loop below)
        const int top = vlo & ~15;                                // 16-byte lines from here down
        bool found = false;
        {
            blk.par([&](int tid) {
                uint32_t key = 0xFFFFFFFFu;
                if (tid == 0)
                    for (int q = vlo - 1; q >= top && key == 0xFFFFFFFFu; --q) {
                        const uint32_t b = ldg(a.text + q);
                        if ((b != 0x0Au && b != 0x0Du) || is_docstart_global(a, q)) key = 0x7FFFFFFEu - static_cast<uint32_t>(q);
                    }
                sm.scan[tid] = key;
            });
            const uint32_t m = blk.reduce_min(sm.scan);
            if (m != 0xFFFFFFFFu) { answer = static_cast<int>(0x7FFFFFFEu - m); found = true; }
        }
        for (int base = top; !found; base -= 64 * kThreads) {
            if (base <= 0) { answer = -1; break; }
            blk.par([&](int tid) {
                // sixty-four bytes a thread, a 16-byte line at a time, downwards
                uint32_t key = 0xFFFFFFFFu;                        // smallest key = highest position that ends the walk
                for (int c = 0; c < 4 && key == 0xFFFFFFFFu; ++c) {
                    const int hi = base - 64 * tid - 16 * c;       // the line is [hi - 16, hi)
                    if (hi <= 0) { key = 0x7FFFFFFFu; break; }    // (position -1)
                    if (hi >= 32 && no_docstart_in16(a, hi - 16)) {
                        const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + hi - 16);
                        const uint32_t v0 = ldg(p4), v1 = ldg(p4 + 1), v2 = ldg(p4 + 2), v3 = ldg(p4 + 3);
                        if (all_bytes_in(v0, 0x0Au, 0x0Du) && all_bytes_in(v1, 0x0Au, 0x0Du) && all_bytes_in(v2, 0x0Au, 0x0Du) && all_bytes_in(v3, 0x0Au, 0x0Du)) continue;
                    }
                    for (int q = hi - 1; q >= hi - 16 && key == 0xFFFFFFFFu; --q) {
                        if (q < 0) { key = 0x7FFFFFFFu; break; }
                        const uint32_t b = ldg(a.text + q);
                        if ((b != 0x0Au && b != 0x0Du) || is_docstart_global(a, q)) key = 0x7FFFFFFEu - static_cast<uint32_t>(q);
                    }
                }
                sm.scan[tid] = key;
            });
            const uint32_t m = blk.reduce_min(sm.scan);
            if (m != 0xFFFFFFFFu) { answer = m == 0x7FFFFFFFu ? -1 : static_cast<int>(0x7FFFFFFEu - m); break; }
        }
        blk.par([&](int tid) { if (tid == 0) sm.far_run[3] = answer; });
    }
}

// One tile of pre-tokenization.
template <bool kWide, class Blk>
GTOK_DEV void pretok_tile(Blk& blk, const EncodeArgs& a, PretokSmem& sm, int tile) {
    const int n = static_cast<int>(ldg(a.meta));
    const int t0 = tile * kPTile;
    const int lo = t0 - kHaloL;
    const uint32_t family = a.tb.family;
    const int n_chunks = kPWin / 16;
    // Diagnostics only: cycles between phase ends, block-summed into phase_clk[slot].
    auto mark = [&](int slot) {
        if (!a.phase_clk) return;
        blk.par([&](int tid) {
            if (tid != 0) return;
            unsigned long long t = cycle_now();
            if (slot >= 0) add_cycles(a.phase_clk + slot, t - sm.clk_last);
            sm.clk_last = t;
#if defined(__CUDA_ARCH__)
            if (sm.misc[2] < 2u && blockIdx.x < kTlBlocks) {
                unsigned long long ns;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
                a.phase_clk[kPhaseWords + (static_cast<size_t>(4 + sm.misc[2]) * kTlBlocks + blockIdx.x) * kTlSlots + (slot + 1)] = ns;
            }
#endif
        });
    };
    mark(-1);

    // ---- P0/P1: each thread fetches 16 bytes and classifies them at once ----
    // Text, per-byte class and flags, the one-hot byte and the chunk's entries of the nine bit
    // planes go to shared memory together; nothing here reads what another thread writes.
    // ASCII and continuation bytes through the 256-entry table, the lead bytes of longer sequences
    // decoded leniently (src/pretok_boundary.h:43-57: the lead byte decides the width when that
    // many bytes remain in the document, anything else is a one-byte codepoint) and looked up in
    // the block's copy of the class table.
    blk.par([&](int tid) {
        if (tid == 0) { sm.misc[1] = 0; sm.misc[3] = 0; sm.far_run[0] = -2; sm.far_run[2] = -2; }
        if (tid < static_cast<int>(sizeof(sm.dirty) / 4)) sm.dirty[tid] = 0;
        for (int wd = tid; wd < kPWin / 32 + 2; wd += kThreads) {
            int gw = (lo >> 5) + wd;                 // lo is a multiple of 32
            uint32_t v = 0;
            if (gw >= 0 && gw * 32 < n) {
                if (a.docmask) v = ldg(a.docmask + gw);
                if (gw == 0) v |= 1u;
            }
            sm.dsw[wd] = v;
        }
        // both of the thread's chunks are requested before either is looked at
        uint32_t both[kPChunks / kThreads][4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int h = 0; h < kPChunks / kThreads; ++h) {
            const int p0 = lo + (tid + h * kThreads) * 16;
            both[h][0] = both[h][1] = both[h][2] = both[h][3] = 0;
            if (p0 >= 0 && p0 < n) {
#if defined(__CUDA_ARCH__)
                const uint4 v = ld128(reinterpret_cast<const uint4*>(a.text + p0));
                both[h][0] = v.x; both[h][1] = v.y; both[h][2] = v.z; both[h][3] = v.w;
#else
                for (int k = 0; k < 16; ++k) both[h][k >> 2] |= static_cast<uint32_t>(a.text[p0 + k]) << (8 * (k & 3));
#endif
            }
        }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int h = 0; h < kPChunks / kThreads; ++h) {
            const int c = tid + h * kThreads;
            const int i0 = c * 16, p0 = lo + i0;
            uint32_t tw[4] = {both[h][0], both[h][1], both[h][2], both[h][3]}, aw[4], ow[4];
            if (p0 + 16 <= 0 || p0 >= n) {
                // wholly outside the text
                uint32_t* txw = reinterpret_cast<uint32_t*>(sm.txt + i0);
                uint32_t* atw = reinterpret_cast<uint32_t*>(sm.attr + i0);
                uint32_t* ohw = reinterpret_cast<uint32_t*>(sm.oh + i0);
                for (int k = 0; k < 4; ++k) { txw[k] = 0; atw[k] = A_OUT * 0x01010101u; ohw[k] = 0; }
                for (int k = 0; k < kPlanes; ++k) sm.plane[k][c] = 0;
                if (kWide) for (int k = 0; k < kXPlanes; ++k) xplane(sm, k)[c] = 0;
                sm.cand16[c] = 0;
                continue;
            }
            uint32_t ds = 0;
            {
                const int gw = p0 >> 5;
                if (gw >= 0 && gw * 32 < n) {
                    uint32_t v = a.docmask ? ldg(a.docmask + gw) : 0u;
                    if (gw == 0) v |= 1u;
                    ds = (v >> (p0 & 31)) & 0xFFFFu;
                }
            }
            uint32_t slow = 0;                                  // lead bytes of multi-byte sequences, decoded below
            uint32_t cand = 0;                                  // bytes that open an added-token literal
            if (p0 >= 0 && p0 + 16 <= n) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
                for (int j = 0; j < 4; ++j) {
                    const uint32_t t = tw[j];
                    const uint32_t v0 = sm.lut[t & 0xFFu], v1 = sm.lut[(t >> 8) & 0xFFu], v2 = sm.lut[(t >> 16) & 0xFFu], v3 = sm.lut[t >> 24];
                    aw[j] = (v0 & 0xFFu) | ((v1 & 0xFFu) << 8) | ((v2 & 0xFFu) << 16) | ((v3 & 0xFFu) << 24);
                    ow[j] = ((v0 >> 8) & 0xFFu) | (v1 & 0xFF00u) | ((v2 & 0xFF00u) << 8) | ((v3 & 0xFF00u) << 16);
                    cand |= (((v0 >> 16) & 1u) | ((v1 >> 15) & 2u) | ((v2 >> 14) & 4u) | ((v3 >> 13) & 8u)) << (4 * j);
                    const uint32_t lead = t & (t << 1) & 0x80808080u;       // bytes 11xxxxxx
                    slow |= (((lead >> 7) * 0x00204081u) >> 21 & 0xFu) << (4 * j);
                }
            } else {
                for (int j = 0; j < 4; ++j) {
                    uint32_t av = 0, ov = 0;
                    for (int k = 0; k < 4; ++k) {
                        const int i = j * 4 + k, p = p0 + i;
                        const uint32_t bt = (tw[j] >> (8 * k)) & 0xFFu;
                        uint32_t at = A_OUT, oh = 0;
                        if (p >= 0 && p < n) {
                            const uint32_t v = sm.lut[bt];
                            at = v & 0xFFu; oh = (v >> 8) & 0xFFu;
                            cand |= ((v >> 16) & 1u) << i;
                            if (bt >= 0xC0u) slow |= 1u << i;
                        }
                        av |= at << (8 * k);
                        ov |= oh << (8 * k);
                    }
                    aw[j] = av;
                    ow[j] = ov;
                }
            }
            uint32_t* txw = reinterpret_cast<uint32_t*>(sm.txt + i0);
            uint32_t* atw = reinterpret_cast<uint32_t*>(sm.attr + i0);
            uint32_t* ohw = reinterpret_cast<uint32_t*>(sm.oh + i0);
#if defined(__CUDA_ARCH__)
            *reinterpret_cast<uint4*>(txw) = make_uint4(tw[0], tw[1], tw[2], tw[3]);
            *reinterpret_cast<uint4*>(atw) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
            *reinterpret_cast<uint4*>(ohw) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
#else
            for (int k = 0; k < 4; ++k) { txw[k] = tw[k]; atw[k] = aw[k]; ohw[k] = ow[k]; }
#endif
            if (ds | slow) {
                // the rarer bytes are put right in shared memory (this thread's own chunk)
                for (uint32_t d = ds; d;) {
                    const int i = ffs32(d);
                    d &= d - 1;
                    sm.attr[i0 + i] |= A_DOC;
                }
                while (slow) {
                    const int i = ffs32(slow);
                    slow &= slow - 1;
                    const int p = p0 + i;
                    const uint32_t b = sm.txt[i0 + i];
                    int avail = n - p;
                    if (avail > 4) avail = 4;
                    if (a.docmask) for (int k = 1; k < avail; ++k) if (is_docstart_global(a, p + k)) { avail = k; break; }
                    const uint32_t b1 = avail > 1 ? ldg(a.text + p + 1) : 0u, b2 = avail > 2 ? ldg(a.text + p + 2) : 0u, b3 = avail > 3 ? ldg(a.text + p + 3) : 0u;
                    uint32_t cp = b;
                    if ((b & 0xE0u) == 0xC0u && avail >= 2) cp = ((b & 0x1Fu) << 6) | (b1 & 0x3Fu);
                    else if ((b & 0xF0u) == 0xE0u && avail >= 3) cp = ((b & 0x0Fu) << 12) | ((b1 & 0x3Fu) << 6) | (b2 & 0x3Fu);
                    else if ((b & 0xF8u) == 0xF0u && avail >= 4) cp = ((b & 0x07u) << 18) | ((b1 & 0x3Fu) << 12) | ((b2 & 0x3Fu) << 6) | (b3 & 0x3Fu);
                    uint32_t cls = A_O;
                    if (kWide) {
                        cls = uc_class([&](uint32_t k) { return static_cast<uint32_t>(ldg(a.tb.uc_stage1 + k)); }, [&](uint32_t k) { return ldg(a.tb.uc_stage2 + k); }, cp, true);
                        if (cp_is_cjk(cp)) cls |= A_CJK;
                    } else if (cp < 0x10000u) {
                        const uint32_t leaf = sm.ucs1[cp >> 7];
                        cls = (sm.ucs2[leaf * 8u + ((cp & 127u) >> 4)] >> ((cp & 15u) * 2u)) & 3u;
                    } else if (cp <= 0x10FFFFu) {
                        const uint32_t leaf = ldg(a.tb.uc_stage1 + (cp >> 7));
                        cls = (ldg(a.tb.uc_stage2 + leaf * 8u + ((cp & 127u) >> 4)) >> ((cp & 15u) * 2u)) & 3u;
                    }
                    sm.attr[i0 + i] = static_cast<uint8_t>(cls | (sm.attr[i0 + i] & A_DOC));
                    sm.oh[i0 + i] = onehot_of(static_cast<uint8_t>(cls & A_CLS));
                }
                ow[0] = ohw[0]; ow[1] = ohw[1]; ow[2] = ohw[2]; ow[3] = ohw[3];
                if (kWide) { aw[0] = atw[0]; aw[1] = atw[1]; aw[2] = atw[2]; aw[3] = atw[3]; }
            }
            chunk_planes(sm, c, ow, tw);
            if (kWide) chunk_xplanes(sm, c, aw, tw);
            sm.cand16[c] = static_cast<uint16_t>(cand);
        }
    });

    mark(1);
    auto byte_any = [&](int q) -> uint32_t {
        int i = q - lo;
        return (i >= 0 && i < kPWin) ? sm.txt[i] : ldg(a.text + q);
    };
    // ---- P2: paint added-token literals ----
    // A literal can only start at a byte that opens one and is followed by a byte that is second in
    // one (two 256-bit sets that come with the tables).  The few such places of a tile are listed,
    // then every (place, literal length) is looked up by a thread of its own -- a single thread
    // going through all lengths of a thirty-byte literal would hold up the whole block for as long
    // as the rest of the tile program takes -- and the longest hit of each place is painted.
    if (a.tb.added_max_bytes) {
        auto paint = [&](int i, uint32_t ml, uint32_t id) {
            const int p = lo + i;
            // the id goes to the literal's slot at once, so that the next kernel need not match again
            if (a.stage && p >= t0 && p < t0 + kPTile) a.stage[p] = id;
            sm.attr[i] = static_cast<uint8_t>(A_ADDED | (sm.attr[i] & A_DOC));
            sm.oh[i] = kOhAdded;
            for (uint32_t j = 1; j < ml && i + static_cast<int>(j) < kPWin; ++j) {
                sm.attr[i + j] = static_cast<uint8_t>(A_CONT | (sm.attr[i + j] & A_DOC));
                sm.oh[i + j] = kOhC | kOhAdded;          // both bits: inside a literal
            }
            const int c_last = (i + static_cast<int>(ml) - 1 < kPWin ? i + static_cast<int>(ml) - 1 : kPWin - 1) >> 4;
            for (int cc = i >> 4; cc <= c_last; ++cc) shared_or(&sm.dirty[cc >> 5], 1u << (cc & 31));
            sm.misc[1] = 1;
        };
        const bool hashed = a.tb.lit_n_lens != 0;
        blk.par([&](int tid) {
            for (int c = tid; c < n_chunks; c += kThreads) {
                uint32_t cand = sm.cand16[c];
                while (cand) {
                    const int k = ffs32(cand);
                    cand &= cand - 1;
                    const int i = c * 16 + k, p = lo + i;
                    if (p < 0 || p >= n) continue;
                    if (!a.tb.lit_single) {                 // every literal has a second byte: it must follow
                        if (p + 1 >= n) continue;
                        const uint32_t b2 = byte_any(p + 1);
                        if (!((a.tb.lit2_bits[b2 >> 5] >> (b2 & 31)) & 1u)) continue;
                    }
                    if (hashed) {
                        const uint32_t slot = shared_add(&sm.misc[3], 1u);
                        if (slot < static_cast<uint32_t>(kLitPlaces)) { sm.lit_at[slot] = static_cast<uint16_t>(i); sm.lit_best[slot] = 0ull; continue; }
                    }
                    // (no hashed table for this vocabulary, or more places than the list holds: one thread, start to end)
                    uint32_t id;
                    uint32_t ml;
                    if (hashed) {
                        const LitView lv{a.tb.littab, sm.lit_lens, a.tb.lit_mask, a.tb.lit_n_lens, a.tb.added_max_bytes};
                        ml = literal_in_window(lv, sm.txt, lo, a.text, a.docmask, p, n, &id);
                    } else ml = match_literal(a, p, n, byte_any, &id);
                    if (ml) paint(i, ml, id);
                }
            }
        });
        uint32_t n_places = sm.misc[3];
        if (n_places > static_cast<uint32_t>(kLitPlaces)) n_places = kLitPlaces;
        if (n_places) {
            const LitView lv{a.tb.littab, sm.lit_lens, a.tb.lit_mask, a.tb.lit_n_lens, a.tb.added_max_bytes};
            auto is_doc = [&](int q) -> bool { return is_docstart_global(a, q); };
            blk.par([&](int tid) {
                for (uint32_t item = tid; item < n_places * lv.n_lens; item += kThreads) {
                    const uint32_t place = item / lv.n_lens, len = lv.lens[item % lv.n_lens];
                    const int i = sm.lit_at[place], p = lo + i;
                    if (len > lit_limit(lv, a.docmask != nullptr, p, n, is_doc)) continue;
                    uint32_t h = 0, pk = kLitHashK;
                    for (uint32_t j = 0; j < len; ++j) { h += byte_any(p + static_cast<int>(j)) * pk; pk *= kLitHashK; }
                    const uint32_t id = lit_lookup(lv, h, len, p, byte_any);
                    if (id != kNoToken) shared_max64(&sm.lit_best[place], (static_cast<unsigned long long>(len) << 32) | id);
                }
            });
            blk.par([&](int tid) {
                if (static_cast<uint32_t>(tid) >= n_places) return;
                const unsigned long long best = sm.lit_best[tid];
                if (best) paint(sm.lit_at[tid], static_cast<uint32_t>(best >> 32), static_cast<uint32_t>(best));
            });
        }
        mark(2);
        if (sm.misc[1]) {
            // the planes of the chunks a literal was painted over
            blk.par([&](int tid) {
                for (int c = tid; c < n_chunks; c += kThreads) {
                    if (!((sm.dirty[c >> 5] >> (c & 31)) & 1u)) continue;
                    const uint32_t* owp = reinterpret_cast<const uint32_t*>(sm.oh + c * 16);
                    const uint32_t* twp = reinterpret_cast<const uint32_t*>(sm.txt + c * 16);
                    const uint32_t ow[4] = {owp[0], owp[1], owp[2], owp[3]}, tw[4] = {twp[0], twp[1], twp[2], twp[3]};
                    chunk_planes(sm, c, ow, tw);
                    if (kWide) {
                        const uint32_t* awp = reinterpret_cast<const uint32_t*>(sm.attr + c * 16);
                        const uint32_t aw[4] = {awp[0], awp[1], awp[2], awp[3]};
                        chunk_xplanes(sm, c, aw, tw);
                    }
                }
            });
        }
    }

    mark(3);
    Win w;
    w.sm = &sm; w.a = &a; w.lo = lo; w.n = n;
    w.vlo = lo < 0 ? 0 : lo + static_cast<int>(a.tb.added_max_bytes);
    w.vhi = lo + kPWin < n ? lo + kPWin : n;
    {
        // (only when the window ends in whitespace or begins with newlines: every thread sees that without a barrier)
        const uint32_t last_b = w.vhi - 1 >= w.vlo ? sm.txt[w.vhi - 1 - lo] : 0u, first_b = w.vlo < w.vhi ? sm.txt[w.vlo - lo] : 0u;
        const bool fwd = w.vhi < n && (last_b == 0x20u || last_b == 0x09u || last_b == 0x0Bu || last_b == 0x0Cu);
        const bool back = w.vlo >= 2 && (first_b == 0x0Au || first_b == 0x0Du);
        if (!a.tb.added_ws && (fwd || back)) far_runs(blk, a, sm, lo, w.vlo, w.vhi, n);
    }

    // ---- P3: boundary bits, 32 bytes per thread as 64-bit planes with 16-bit margins ----
    // Bit i of a plane is byte i; "<< 1" moves a fact from a byte to the byte after it.
    // Cases the plane algebra does not cover are marked uncertain and decided one by one
    // by is_boundary(): anything within three bytes after an apostrophe (contractions),
    // plain whitespace right after a newline (needs run walks), and words holding stray
    // continuation bytes or added-token literals.
    blk.par([&](int tid) {
        if (tid >= kPTileWords) return;
        const int ww = kHaloL / 32 + tid;
        auto load = [&](int k) -> uint64_t {
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(sm.plane[k]);
            return (static_cast<uint64_t>(pw[ww - 1]) >> 16) | (static_cast<uint64_t>(pw[ww]) << 16) | (static_cast<uint64_t>(pw[ww + 1]) << 48);
        };
        const uint64_t OWN = 0x0000FFFFFFFF0000ull;
        const uint64_t L = load(PL_L), N = load(PL_N), S = load(PL_S), O = load(PL_O), C = load(PL_C), ADraw = load(PL_AD);
        const uint64_t AD = ADraw & ~C;      // first byte of an added-token literal; ADraw & C marks its other bytes
        const uint64_t CR = load(PL_CRLF), SP = load(PL_SP), AP = load(PL_AP);
        const uint64_t DOC = (static_cast<uint64_t>(sm.dsw[ww - 1]) >> 16) | (static_cast<uint64_t>(sm.dsw[ww]) << 16) | (static_cast<uint64_t>(sm.dsw[ww + 1]) << 48);
        const uint64_t LEAD = L | N | S | O | AD;
        auto fill = [&](uint64_t x) -> uint64_t {      // spread a lead's bit over its continuation bytes
            x |= (x << 1) & C; x |= (x << 1) & C; x |= (x << 1) & C;
            return x;
        };
        auto prevcp = [&](uint64_t x) -> uint64_t {    // at each lead: x of the codepoint before it (0 at a document start)
            return (fill(x) << 1) & LEAD & ~DOC;
        };
        auto nextcp = [&](uint64_t x) -> uint64_t {    // at each lead: x of the codepoint after it (0 at a document end)
            uint64_t y = (x & ~DOC) >> 1;              // lands on the last byte of the codepoint before
            y |= (y & C) >> 1; y |= (y & C) >> 1; y |= (y & C) >> 1;
            return y & LEAD;
        };
        const uint64_t pL = prevcp(L), pN = prevcp(N), pS = prevcp(S), pO = prevcp(O);
        const uint64_t pSP = prevcp(SP), pCR = prevcp(CR);
        const uint64_t pNone = LEAD & ~(pL | pN | pS | pO);
        uint64_t bnd = 0, pend = 0, unc = 0;
        // words the algebra cannot be trusted on
        // (a continuation byte right after an apostrophe stretches a contraction past three bytes)
        // An added-token literal is its start bit plus continuation bits; those long stretches are
        // harmless to the algebra (the literal has no class, so its neighbours see "nothing").
        if (kWide && family == 4) {
            // Gemma-3 shape: every byte outside an added-token literal is decided one by one (is_boundary_sp)
            unc = ~(ADraw & C);
            for (int bit = 16; bit < 48; ++bit) {
                const int p = lo + ww * 32 + bit - 16;
                if (p < 0 || p >= n) unc &= ~(1ull << bit);
            }
        } else if (kWide) {
            // DeepSeek-V3 (see is_boundary_deepseek for the rules; here the same over whole planes).
            auto xload = [&](int k) -> uint64_t {
                const uint32_t* pw = reinterpret_cast<const uint32_t*>(xplane(sm, k));
                return (static_cast<uint64_t>(pw[ww - 1]) >> 16) | (static_cast<uint64_t>(pw[ww]) << 16) | (static_cast<uint64_t>(pw[ww + 1]) << 48);
            };
            const uint64_t PS = xload(XP_PS), AL = xload(XP_AL), APU = xload(XP_APU), CJ = xload(XP_CJK);
            const uint64_t Op = O & ~PS;                        // the O plane holds punctuation and symbols too
            const uint64_t Cg = C & ~ADraw;
            const bool messy = (Cg & (Cg << 1) & (Cg << 2) & (Cg << 3)) != 0 || (DOC & C) != 0;
            const uint64_t pPS = prevcp(PS), pOp = prevcp(Op), pCJ = prevcp(CJ), pAL = prevcp(AL), pAPU = prevcp(APU);
            // ends of the pieces the first two patterns leave: numbers, and changes into or out of the CJK ranges
            const uint64_t up = pNone | N | pN | ((CJ ^ pCJ) & LEAD);
            const uint64_t in = LEAD & ~up;                     // the codepoint before is in this one's piece
            bnd |= AD | (DOC & C) | pNone | (N & ~pN) | (~N & pN & LEAD) | ((CJ ^ pCJ) & LEAD & ~N);
            pend = N & pN;
            const uint64_t nIn = nextcp(in);                    // the codepoint after is in this one's piece
            const uint64_t nL = nextcp(L & in), nNonS = nextcp((L | PS | Op) & in);
            (void)nIn;
            // a punctuation mark that takes the ASCII letters after it along: not inside or behind other punctuation
            const uint64_t blocked = (pPS | pSP) & in;
            const uint64_t takes = L & AL & in & pAPU & ~prevcp(blocked);
            bnd |= L & in & ((pS & pCR) | (pPS & ~takes));
            // ASCII letters that such a mark took along end where another kind of letter follows: one by one
            unc |= L & in & pL & pAL & ~AL;
            bnd |= PS & in & ~(pPS | pSP);
            const uint64_t Scr = S & CR, Spl = S & ~CR;
            bnd |= Scr & in & (pL | pOp);
            bnd |= Spl & in & ~pS;
            bnd |= Spl & in & pS & ~pCR & nNonS;
            const uint64_t cand = Spl & in & pS & pCR;
            if (cand) {
                const uint64_t Mcr = CR & ~DOC;
                const uint64_t rs = CR & (~(CR << 1) | DOC);
                const uint64_t absorbed = ((Mcr + (rs & pPS & in & Mcr)) ^ Mcr) & Mcr;
                const uint64_t from_edge = (Mcr & 1ull) ? (((Mcr + 1ull) ^ Mcr) & Mcr) : 0ull;
                const uint64_t SplF = fill(Spl) & ~DOC;
                const uint64_t top_nl = SplF & ((CR & ~DOC) >> 1);
                const uint64_t rM = brev64(SplF), rT = brev64(top_nl);
                const uint64_t later_nl = brev64(((rM + rT) ^ rM) & rM);
                const uint64_t to_edge = (rM & 1ull) ? brev64(((rM + 1ull) ^ rM) & rM) : 0ull;
                const uint64_t unknown = cand & ((from_edge << 1) | to_edge);
                bnd |= cand & ~unknown & ((absorbed << 1) | ~later_nl);
                unc |= unknown;
            }
            bnd |= Op & in & (~pOp | nL);
            if (messy) unc = LEAD;
        } else {
            const uint64_t Cg = C & ~ADraw;
            // (a stray continuation byte right after an apostrophe is glued to it and pushes the tail letters along)
            // (DeepSeek-V3: every codepoint is decided one by one from the attribute bytes)
            const bool messy = (Cg & (Cg << 1) & (Cg << 2) & (Cg << 3)) != 0 || (DOC & C) != 0 || ((AP << 1) & C) != 0;
            if (messy) unc = LEAD;
            // An apostrophe with a continuation byte within the three bytes after it: what follows is not
            // plain ASCII (U+017F counts as 's'), so this apostrophe and the three bytes after it, where a
            // contraction and the letter after it would lie, are decided one by one; the word's other
            // apostrophes stay with the algebra.
            const uint64_t apC = AP & ((C >> 1) | (C >> 2) | (C >> 3));
            // Contractions: 's 't 'm 'd (tail 1) and 're 've 'll (tail 2), when the regex cursor can be
            // at the apostrophe (anything but punctuation or a literal space before it).  The few
            // apostrophes of a word are looked at one by one; what follows them is ASCII or the case
            // goes to the one-by-one path.
            uint64_t cs1 = 0, cs2 = 0;
            if (!messy && AP) {
                const bool ci = family != 0;
                uint64_t aps = AP & LEAD & ~(pO | pSP) & ~apC;
                while (aps) {
    #if defined(__CUDA_ARCH__)
                    const int bit = __ffsll(static_cast<long long>(aps)) - 1;
    #else
                    const int bit = __builtin_ctzll(aps);
    #endif
                    aps &= aps - 1;
                    const uint64_t m = 1ull << bit;
                    if (bit > 59) { unc |= m; continue; }                   // tail would leave the window
                    const int i = ww * 32 + bit - 16;
                    uint32_t x = sm.txt[i + 1], y = sm.txt[i + 2];
                    if (x >= 0x80u || ((DOC >> (bit + 1)) & 3u)) { unc |= (m | (m << 1) | (m << 2) | (m << 3) | (m << 4)) & LEAD; continue; }
                    if (ci) { if (x >= 'A' && x <= 'Z') x += 32; if (y >= 'A' && y <= 'Z') y += 32; }
                    // the second letter must be a letter of this document too (an added-token literal is not)
                    const bool y_ok = ((L >> (bit + 2)) & 1u) != 0;
                    if (!((L >> (bit + 1)) & 1u)) continue;
                    if ((x == 'r' || x == 'v') && y == 'e' && y_ok) cs2 |= m;
                    else if (x == 'l' && y == 'l' && y_ok) cs2 |= m;
                    else if (x == 's' || x == 't' || x == 'm' || x == 'd') cs1 |= m;
                }
            }
            {
                const uint64_t x = messy ? AP : apC;
                unc |= (x | (x << 1) | (x << 2) | (x << 3)) & LEAD;
            }
            bnd |= AD | (DOC & C) | pNone;
            if (family == 0) {
                const uint64_t nNonS = nextcp(L | N | O);
                bnd |= S & (~pS | nNonS);
                const uint64_t rest = (L | N | O) & ~pSP;          // a literal space before leads the token
                bnd |= rest & ((L & ~pL) | (N & ~pN) | (O & ~pO));
            } else {
                const uint64_t nNonS = nextcp(L | N | O);
                const uint64_t Scr = S & CR, Spl = S & ~CR;
                bnd |= Scr & (pL | pN);
                bnd |= Spl & ~pS;
                bnd |= Spl & pS & ~pCR & nNonS;
                // Plain whitespace right after a newline: it opens the rest of the run when the newline
                // stretch before it hangs off a punctuation token, or when no later newline in the run
                // pulls it into \s*[\r\n]+.  Both are floods along a stretch of bits (carry of an
                // addition); a stretch that leaves the window is decided one by one instead.
                const uint64_t cand = Spl & pS & pCR;
                if (cand) {
                    const uint64_t Mcr = CR & ~DOC;                              // newline bytes, stretches cut at document starts
                    const uint64_t rs = CR & (~(CR << 1) | DOC);                 // first byte of each stretch
                    const uint64_t absorbed = ((Mcr + (rs & pO & Mcr)) ^ Mcr) & Mcr;
                    const uint64_t from_edge = (Mcr & 1ull) ? (((Mcr + 1ull) ^ Mcr) & Mcr) : 0ull;   // stretch whose start is not visible
                    const uint64_t SplF = fill(Spl) & ~DOC;
                    const uint64_t top_nl = SplF & ((CR & ~DOC) >> 1);           // whitespace byte directly before a newline
                    const uint64_t rM = brev64(SplF), rT = brev64(top_nl);
                    const uint64_t later_nl = brev64(((rM + rT) ^ rM) & rM);     // whitespace stretches that end in a newline
                    const uint64_t to_edge = (rM & 1ull) ? brev64(((rM + 1ull) ^ rM) & rM) : 0ull;  // stretch that reaches the window's end
                    const uint64_t unknown = cand & ((from_edge << 1) | to_edge);
                    bnd |= cand & ~unknown & ((absorbed << 1) | ~later_nl);
                    unc |= unknown;
                }
                const uint64_t ppOorSP = prevcp(pO | pSP);         // prev-prev is punctuation or a literal space
                bnd |= L & ((pS & pCR) | (pO & ppOorSP) | pN);
                if (family == 2) bnd |= N;
                else { bnd |= N & ~pN; pend = N & pN; }
                bnd |= O & ~pO & ~pSP;
            }
            {
                const uint64_t in_tail = ((cs1 | cs2) << 1) | (cs2 << 2);
                const uint64_t after_tail = (cs1 << 2) | (cs2 << 3);
                bnd = (bnd & ~in_tail) | cs1 | cs2 | (after_tail & L & pL);
            }
        }
        bnd &= ~unc;
        pend &= ~unc;
        uint64_t nstart = N & ~pN;
        // one-by-one decisions
        uint64_t todo = unc & OWN;
        while (todo) {
#if defined(__CUDA_ARCH__)
            const int bit = __ffsll(static_cast<long long>(todo)) - 1;
#else
            const int bit = __builtin_ctzll(todo);
#endif
            todo &= todo - 1;
            const int i = ww * 32 + bit - 16, p = lo + i;
            const uint8_t a0 = sm.attr[i];
            const uint64_t m = 1ull << bit;
            if ((a0 & A_CLS) == A_ADDED) { bnd |= m; continue; }
            if (kWide && family == 4 && i >= 1) {
                // Gemma-3 shape, an ASCII character after an ASCII character of the same document, no added token before it: settled
                // from two bit sets of the vocabulary's ASCII characters (is_boundary_sp says the same, by the long way)
                const uint32_t c = sm.txt[i], c1 = sm.txt[i - 1];
                if (c < 0x80u && c1 < 0x80u && p >= 1 && !((DOC >> bit) & 1ull) && !((ADraw >> (bit - 1)) & 1ull)) {
                    const bool known = (a.tb.sp_ascii_known[c >> 5] >> (c & 31)) & 1u, known1 = (a.tb.sp_ascii_known[c1 >> 5] >> (c1 & 31)) & 1u;
                    const bool cut = !known || !known1 || (c == 0x20u && !((a.tb.sp_ascii_before_bar[c1 >> 5] >> (c1 & 31)) & 1u));
                    if (cut) bnd |= m; else bnd &= ~m;
                    continue;
                }
            }
            bool pending = false, ns = false;
            const bool bb = kWide ? (family == 4 ? is_boundary_sp(w, p) : is_boundary_deepseek(w, p, a0, &pending, &ns)) : is_boundary(w, p, a0, family, &pending, &ns);
            if (bb) bnd |= m; else bnd &= ~m;
            if (pending) pend |= m; else pend &= ~m;
            if ((a0 & A_CLS) == A_N) { if (ns) nstart |= m; else nstart &= ~m; }
        }
        uint32_t* bndw = reinterpret_cast<uint32_t*>(sm.bnd16);
        reinterpret_cast<uint32_t*>(sm.bnd16)[tid] = static_cast<uint32_t>((bnd & OWN) >> 16);
        reinterpret_cast<uint32_t*>(sm.add16)[tid] = static_cast<uint32_t>((AD & OWN) >> 16);
        reinterpret_cast<uint32_t*>(sm.pend16)[tid] = static_cast<uint32_t>((pend & OWN) >> 16);
        reinterpret_cast<uint32_t*>(sm.lead16)[tid] = static_cast<uint32_t>((LEAD & OWN) >> 16);
        reinterpret_cast<uint32_t*>(sm.nlead16)[tid] = static_cast<uint32_t>((N & OWN) >> 16);
        reinterpret_cast<uint32_t*>(sm.nstart16)[tid] = static_cast<uint32_t>((nstart & OWN) >> 16);
        (void)bndw;
    });

    mark(4);
    // ---- P4: index of each digit in its run (\p{N}{1,3} of Llama-3 and DeepSeek-V3) ----
    if (family == 1 || (kWide && family == 3)) {
        const uint32_t* leadw = reinterpret_cast<const uint32_t*>(sm.lead16);
        const uint32_t* nleadw = reinterpret_cast<const uint32_t*>(sm.nlead16);
        const uint32_t* nstartw = reinterpret_cast<const uint32_t*>(sm.nstart16);
        // (has, cnt): "a run start was seen" and "digits since the last run start".
        constexpr int kLaneWords = (kPTileWords + 31) / 32;
        blk.par([&](int tid) {
            if (tid >= 32) return;
            uint32_t has = 0, cnt = 0, last = 0, firstn = 0;
            for (int k = 0; k < kLaneWords; ++k) {
                const int wd = tid * kLaneWords + k;
                if (wd >= kPTileWords) break;
                uint32_t nl = nleadw[wd], st = nstartw[wd];
                if (st) { has = 1; cnt = popc32(nl & ~((1u << fls32(st)) - 1u)); }
                else cnt += popc32(nl);
                if (leadw[wd]) last = wd + 1;
                if (nl && !firstn) firstn = wd + 1;
            }
            sm.sum_has[tid] = has;
            sm.sum_cnt[tid] = cnt;
            sm.lane_last[tid] = last;          // 1 + the lane's last word holding a lead byte, 0 = none
            sm.lane_firstn[tid] = firstn;      // 1 + its first word holding a digit
        });
        blk.par([&](int tid) {
            if (tid != 0) return;
            // Tile summary, published before anything that waits.
            uint32_t has = 0, cnt = 0, any_lead = 0, last_is_n = 0;
            for (int l = 0; l < 32; ++l) {
                if (sm.sum_has[l]) { has = 1; cnt = sm.sum_cnt[l]; } else cnt += sm.sum_cnt[l];
            }
            for (int l = 31; l >= 0; --l) {
                if (sm.lane_last[l]) { const int wd = sm.lane_last[l] - 1; any_lead = 1; last_is_n = (nleadw[wd] >> fls32(leadw[wd])) & 1u; break; }
            }
            bool pass = !any_lead || (last_is_n && !has);     // the run (if any) is still open and began earlier
            uint32_t first_needs = 0;                          // first digit of the tile continues an earlier run
            for (int l = 0; l < 32; ++l) {
                if (sm.lane_firstn[l]) { const int wd = sm.lane_firstn[l] - 1; int b = ffs32(nleadw[wd]); first_needs = !((nstartw[wd] >> b) & 1u); break; }
            }
            unsigned long long mine;
            if (!pass) mine = kStFinal | ((last_is_n && any_lead) ? cnt : 0u);
            else mine = kStAgg | cnt;
            if (tile == 0 && pass) mine = kStFinal | cnt;
            store_state(a.st1 + tile, mine);
            uint32_t carry_in = 0;
            if ((pass || first_needs) && tile > 0) {
                for (int j = tile - 1; j >= 0; --j) {
                    unsigned long long v = wait_state(a.st1, j, a.ctl);
                    carry_in += static_cast<uint32_t>(v);
                    if ((v >> 62) == 2) break;
                }
                if (pass) store_state(a.st1 + tile, kStFinal | (carry_in + cnt));
            }
            sm.misc[0] = carry_in;
        });
        blk.par([&](int tid) {
            if (tid >= 32) return;
            // Exclusive (has, cnt) over the 32 lane summaries, seeded with the carry.
            uint32_t cnt = sm.misc[0];
            for (int l = 0; l < tid; ++l) { if (sm.sum_has[l]) cnt = sm.sum_cnt[l]; else cnt += sm.sum_cnt[l]; }
            for (int k = 0; k < kLaneWords; ++k) {
                const int wd = tid * kLaneWords + k;
                if (wd >= kPTileWords) break;
                sm.carry[wd] = cnt;
                uint32_t nl = nleadw[wd], st = nstartw[wd];
                if (st) cnt = popc32(nl & ~((1u << fls32(st)) - 1u));
                else cnt += popc32(nl);
            }
        });
        blk.par([&](int tid) {
            for (int h = tid; h < 2 * kPTileWords; h += kThreads) {
                uint32_t pend = sm.pend16[h];
                if (!pend) continue;
                int wd = h >> 1, shift = (h & 1) * 16;
                uint32_t nl = nleadw[wd], st = nstartw[wd], bnd = sm.bnd16[h];
                while (pend) {
                    int k = ffs32(pend);
                    pend &= pend - 1;
                    int bit = shift + k;
                    uint32_t below = (1u << bit) - 1u;
                    uint32_t idx;
                    uint32_t st_below = st & below;
                    if (st_below) idx = popc32(nl & below & ~((1u << fls32(st_below)) - 1u));
                    else idx = sm.carry[wd] + popc32(nl & below);
                    if (idx % 3u == 0u) bnd |= 1u << k;
                }
                sm.bnd16[h] = static_cast<uint16_t>(bnd);
            }
        });
    }

    mark(5);
    // ---- P5: write the bit masks, count boundaries ----
    // The masks are arrays of whole 4096-byte tiles' worth of words (what the kernels after this one
    // read, and what a caller's buffer holds): nothing is written past that, and the last tile
    // clears whatever lies between its own end and there.
    {
        const uint32_t lim = static_cast<uint32_t>((n + kTile - 1) / kTile) * kTileWords;
        const bool last = t0 + kPTile >= n;
        blk.par([&](int tid) {
            uint32_t cnt = 0;
            if (tid < kPTileWords) {
                const uint32_t bw = reinterpret_cast<const uint32_t*>(sm.bnd16)[tid];
                const uint32_t idx = static_cast<uint32_t>(tile) * kPTileWords + tid;
                if (idx < lim) {
                    a.bmask[idx] = bw;
                    if (a.tb.added_max_bytes) a.amask[idx] = reinterpret_cast<const uint32_t*>(sm.add16)[tid];
                }
                cnt = popc32(bw);
            }
            if (last) {
                for (uint32_t idx = static_cast<uint32_t>(tile + 1) * kPTileWords + tid; idx < lim; idx += kThreads) {
                    a.bmask[idx] = 0;
                    if (a.tb.added_max_bytes) a.amask[idx] = 0;
                }
            }
            sm.scan[tid] = cnt;
        });
    }
    uint32_t total = 0;
    blk.excl_scan(sm.scan, &total);
    blk.par([&](int tid) { if (tid == 0) a.tile_nb[tile] = total; });
    mark(6);
}

// ==================================================================================
//                                   MERGE + ASSEMBLY
// ==================================================================================
constexpr int kMissBatch = kThreads / 2;       // unknown pre-tokens per batch of the miss kernel
constexpr int kArenaSyms = 3072;               // symbols of one batch (ids, ranks, results: 36 KB)
constexpr int kSumTiles = 16384;               // documents up to this many tiles (64 MiB): tile bases by direct summation
constexpr int kLongPerTile = 64;               // a tile holds fewer than 4096 / 65 pre-tokens longer than 64 bytes
enum { CTL_PRETOK = 0, CTL_ASM = 1, CTL_ERR = 2, CTL_EXIT = 3, CTL_NMISS = 4, CTL_NLONG = 5, CTL_BATCH = 6, CTL_LONG = 7, CTL_NMED = 8, CTL_NFC = 9, CTL_NMED2 = 10, CTL_NMED1 = 11, CTL_NFCFLAG = 12,
       CTL_FILTERED = 13,   // calls of the 17..32-byte class that are through their whole-token lookups (surplus handed back)
       CTL_SURPLUS = 14,    // ticket for the chunks of that surplus
       CTL_NSURPLUS = 15 }; // entries handed back in all
constexpr int kShortWordMax = 16;              // unknown pre-tokens up to this length and the longer ones are batched apart
// A batch lasts as long as its longest merge chain, so pre-tokens are batched by length class and
// the classes are handed out longest first: 49..64 bytes, 33..48, 17..32, then the short ones.
// Batch sizes are such that a batch always fits the arena (48 * 64, 64 * 48, 96 * 32 slots).
constexpr int kMedSplit = 32;
constexpr int kMedSplit1 = 48;
constexpr int kMedBatchA = 48;                 // 49..64 bytes
constexpr int kMedBatchA1 = 64;                // 33..48 bytes
constexpr int kMedBatchB = 96;                 // 17..32 bytes
constexpr int kMedTakeB = kThreads;            // list entries per call of that class under ignore_merges (most are whole tokens)

struct WordsSmem {
    alignas(16) uint8_t txt[kTile + 64];
    uint32_t bm[kTileWords + 4];
    uint32_t am[kTileWords + 4];
    alignas(16) uint32_t tok[kTile + kTokExtra];
    uint16_t wl[kTile + 8];            // offsets in the tile of the pre-token starts, in order; then the end sentinel
    uint32_t miss[kTile / 2];          // offset | len << 12, up to 16 bytes
    uint32_t med[kTile / 16];          // offset | len << 12: 49..64 bytes from the front, 17..32 bytes from the back
    uint32_t med1[kTile / 32];         // offset | len << 12: 33..48 bytes
    uint32_t lng_o[kLongPerTile], lng_len[kLongPerTile];
    uint32_t b2i[256];
    uint32_t scan[kThreads];
    uint32_t ctr[12];
    unsigned long long clk_last;
};
struct MissSmem {
    alignas(16) uint32_t ws[3 * kArenaSyms];   // arena: ids, ranks, results (also the long pre-token workspace)
    uint32_t b2i[256];
    unsigned long long word[kThreads]; // this batch's entries of the global list (0 = none, or done already)
    unsigned long long cand[kThreads]; // list entries left over after the whole-token look-up
    alignas(16) uint16_t lnk[kArenaSyms];   // live-symbol chain of each pre-token (prev << 8 | next)
    alignas(16) uint32_t gmin[kArenaSyms / 4];   // lowest rank key of each group of four slots, laid out like the arena (pre-tokens of more than 16 bytes)
    uint8_t rawb[kArenaSyms];          // the pre-tokens' text bytes, max_len apart
    uint32_t ctr[8];
    unsigned long long clk_last;
};
struct AsmSmem {
    uint32_t scan[kThreads];           // ids in each thread's sixteen slots, then their exclusive sums
    uint32_t sum[kThreads];            // each thread's share of the earlier tiles' id counts
    uint32_t ex[kTokExtra / 4];        // ids in each quad of the tile's overflow slots
    uint32_t ovf[kTokExtra];           // the tile's overflow slots
    uint32_t lref_idx[kLongPerTile], lref_at[kLongPerTile];
    uint32_t ctr[8];
    unsigned long long clk_last;
};
enum { C_NMISS = 0, C_NTEAM = 1, C_BASEM = 2, C_BASEL = 3, C_USED = 4, C_TMP = 5, C_TMP2 = 6, C_NLREF = 7, C_NMED = 5, C_BASED = 6, C_NMED2 = 4, C_BASED2 = 7, C_NKNOWN = 8, C_NMED1 = 9, C_BASED1 = 10 };

// Greedy BPE of one pre-token by a single thread (lowest rank first, leftmost among
// equals, src/host_encode.cc:617-648).  ids/rk/nw are the pre-token's stretch of the
// block's symbol arena with the pair ranks already probed; merged-away symbols are
// marked dead in place, so a step is one pass over the slots plus one round trip for
// the two new pairs.
// What the arena keeps per pair is rank << 6 | slot (kNoRank when no rule joins the pair): the
// lowest key is the lowest rank and, among equal ranks, the leftmost pair, so the search for the
// next merge is a plain minimum.  Ranks stay below 2^26 - 1 (checked when the tables are built),
// slots below 64.
GTOK_DEV uint32_t rank_key(uint32_t rank, uint32_t slot) { return rank == kNoRank ? kNoRank : ((rank << 6) | slot); }

// The arena holds the batch's pre-tokens interleaved by groups of four slots: slot r of
// pre-token w (of W in the batch) is element (r / 4 * W + w) * 4 + r % 4.  The threads of a
// warp own consecutive pre-tokens, so when they all read their group g the 32 loads of 16
// bytes are contiguous in shared memory (no bank conflict), however long each pre-token is.
GTOK_DEV uint32_t arena_at(uint32_t w4, uint32_t stride, uint32_t r) { return (r >> 2) * stride + w4 + (r & 3u); }   // w4 = 4 * w, stride = 4 * W

// ids/rk/nw/lnk are the arena's bases; the pre-token is number w4 / 4 of stride / 4; its k-th id
// goes to the slot array by put(k, id).  Returns the number of ids.
// For a pre-token of more than 16 bytes the search for the lowest key goes through gm, the lowest key
// of each group of four slots (same interleaved layout, so four groups are one 128-bit load): a
// step reads a quarter of what a pass over all slots would and then puts right the three groups the
// merge touched.  The search is half of what a step costs beside its one memory round trip.
// `hist` is told whenever the pre-token's first or last symbol changes (the new symbol and the rank of
// the merge that made it): what pieces_word needs to know about a piece's two ends.
struct NoEdgeHistory {
    GTOK_DEV void first(uint32_t, uint32_t) {}
    GTOK_DEV void last(uint32_t, uint32_t) {}
};
template <class Put, class Hist = NoEdgeHistory>
GTOK_DEV uint32_t bpe_arena(const EncodeArgs& a, uint32_t* ids, uint32_t* rk, uint32_t* nw, uint16_t* lnk, uint32_t* gm, uint32_t w4, uint32_t stride,
                            uint32_t len, Put put, Hist hist = Hist()) {
    // lnk[slot] = prev << 8 | next (slot numbers within the pre-token, 0xFF = none) keeps the
    // live symbols chained; slots past `len` in the last group hold no rank.
    const uint32_t groups = (len + 3u) >> 2;
    const bool two_level = len > 16u;
    auto group_min = [&](uint32_t g) -> uint32_t {
#if defined(__CUDA_ARCH__)
        const uint4 v = reinterpret_cast<const uint4*>(rk + w4)[g * (stride >> 2)];
        return min(min(v.x, v.y), min(v.z, v.w));
#else
        uint32_t m = kNoRank;
        for (uint32_t r = g * 4; r < g * 4 + 4; ++r) { const uint32_t v = rk[arena_at(w4, stride, r)]; if (v < m) m = v; }
        return m;
#endif
    };
    for (;;) {
        uint32_t best = kNoRank;
        if (two_level) {
            const uint32_t quads = (groups + 3u) >> 2;
#if defined(__CUDA_ARCH__)
            const uint4* gp = reinterpret_cast<const uint4*>(gm + w4);
            const uint32_t gs = stride >> 2;
#pragma unroll 4
            for (uint32_t q = 0; q < quads; ++q) {
                const uint4 v = gp[q * gs];
                best = min(best, min(min(v.x, v.y), min(v.z, v.w)));
            }
#else
            for (uint32_t g = 0; g < quads * 4; ++g) { const uint32_t v = gm[arena_at(w4, stride, g)]; if (v < best) best = v; }
#endif
        } else {
#if defined(__CUDA_ARCH__)
            const uint4* rp = reinterpret_cast<const uint4*>(rk + w4);
            const uint32_t gs = stride >> 2;
#pragma unroll 4
            for (uint32_t g = 0; g < groups; ++g) {
                const uint4 v = rp[g * gs];
                best = min(best, min(min(v.x, v.y), min(v.z, v.w)));
            }
#else
            for (uint32_t r = 0; r < groups * 4; ++r) { const uint32_t v = rk[arena_at(w4, stride, r)]; if (v < best) best = v; }
#endif
        }
        if (best == kNoRank) break;
        const uint32_t bi = best & 63u, xb = arena_at(w4, stride, bi);
        const uint32_t l = lnk[xb];
        const uint32_t j = l & 0xFFu, p = l >> 8;
        const uint32_t xj = arena_at(w4, stride, j);
        const uint32_t k = lnk[xj] & 0xFFu;
        const uint32_t merged = nw[xb];
        ids[xb] = merged;
        if (p == 0xFFu) hist.first(merged, best >> 6);
        if (k == 0xFFu) hist.last(merged, best >> 6);
        rk[xj] = kNoRank;
        lnk[xb] = static_cast<uint16_t>((p << 8) | k);
        const uint32_t xk = arena_at(w4, stride, k & 63u), xp = arena_at(w4, stride, p & 63u);
        if (k != 0xFFu) lnk[xk] = static_cast<uint16_t>((bi << 8) | (lnk[xk] & 0xFFu));
        RankRes right, left;
        probe_rule2(a.tb, k != 0xFFu, merged, k != 0xFFu ? ids[xk] : 0u, &right, p != 0xFFu, p != 0xFFu ? ids[xp] : 0u, merged, &left);
        rk[xb] = rank_key(right.rank, bi); nw[xb] = right.res;
        if (p != 0xFFu) { rk[xp] = rank_key(left.rank, p); nw[xp] = left.res; }
        if (two_level) {
            const uint32_t gb = bi >> 2, gj = j >> 2;
            gm[arena_at(w4, stride, gb)] = group_min(gb);
            if (gj != gb) gm[arena_at(w4, stride, gj)] = group_min(gj);
            if (p != 0xFFu && (p >> 2) != gb) gm[arena_at(w4, stride, p >> 2)] = group_min(p >> 2);
        }
    }
    uint32_t c = 0;
    for (uint32_t i = 0; i != 0xFFu;) {
        const uint32_t x = arena_at(w4, stride, i);
        put(c++, ids[x]);
        i = lnk[x] & 0xFFu;
    }
    return c;
}

// Team (warp or whole block) BPE over arrays ids/rk/nw of n symbols, which may live
// in shared or global memory.  `Team` supplies:
//     kSize, par(f), excl_scan(arr[kSize], &total), reduce_min(arr[kSize]) -> value
//     keep(lane, k)   three words per lane that survive from one par() to the next
// and `scratch` is shared memory of at least 3*kSize + 16 words owned by the team.
//
// For vocabularies whose rule ranks are monotone (a rule's operands are made by
// earlier rules only) all pairs of the current lowest rank are merged in one
// round: a merge can then only create pairs of higher rank, so the set of
// lowest-rank pairs is fixed for the round, and the only interaction among them
// is inside a stretch of overlapping equal pairs (x x x x ...), where the greedy
// left-to-right order takes every other pair starting from the left.
// Otherwise one merge is applied per round, exactly as the scalar loop would.
template <class Team>
GTOK_DEV uint32_t team_bpe(Team& tm, const EncodeArgs& a, uint32_t* ids, uint32_t* rk, uint32_t* nw, uint32_t n, uint32_t* scratch) {
    constexpr int T = Team::kSize;
    uint32_t* s_a = scratch;            // [T]
    uint32_t* s_b = scratch + T;        // [T]
    uint32_t* s_c = scratch + 2 * T;    // [T]
    uint32_t* s_m = scratch + 3 * T;    // [T / 32 + 1]
    tm.par([&](int lane) {
        for (uint32_t i = lane; i < n; i += T) {
            if (i + 1 < n) { RankRes r = probe_rule(a.tb, ids[i], ids[i + 1]); rk[i] = r.rank; nw[i] = r.res; }
            else { rk[i] = kNoRank; nw[i] = 0; }
        }
    });
    for (;;) {
        if (n < 2) break;
        tm.par([&](int lane) {
            uint32_t best = kNoRank;
            for (uint32_t i = lane; i < n; i += T) { uint32_t r = rk[i]; if (r < best) best = r; }
            s_a[lane] = best;
        });
        const uint32_t m = tm.reduce_min(s_a);
        if (m == kNoRank) break;
        if (!a.tb.monotone) {
            // One merge, by lane 0: the leftmost pair of rank m.
            tm.par([&](int lane) {
                if (lane != 0) return;
                uint32_t bi = 0;
                while (rk[bi] != m) ++bi;
                ids[bi] = nw[bi];
                for (uint32_t i = bi + 1; i + 1 < n; ++i) { ids[i] = ids[i + 1]; rk[i] = rk[i + 1]; nw[i] = nw[i + 1]; }
                uint32_t nn = n - 1;
                rk[nn - 1] = kNoRank;
                if (bi + 1 < nn) { RankRes r = probe_rule(a.tb, ids[bi], ids[bi + 1]); rk[bi] = r.rank; nw[bi] = r.res; }
                else rk[bi] = kNoRank;
                if (bi > 0) { RankRes r = probe_rule(a.tb, ids[bi - 1], ids[bi]); rk[bi - 1] = r.rank; nw[bi - 1] = r.res; }
            });
            --n;
            continue;
        }
        // ---- one round: merge every selected pair of rank m, compacting in place ----
        uint32_t out_base = 0;      // symbols written so far
        uint32_t carry_run = 0;     // length of the stretch of rank-m pairs ending just before this chunk
        uint32_t prev_sel = 0;      // was the last element of the previous chunk a selected pair
        for (uint32_t base = 0; base < n; base += T) {
            // (a) flags
            tm.par([&](int lane) {
                uint32_t e = base + lane;
                s_a[lane] = (e < n && rk[e] == m) ? 1u : 0u;
            });
            // (b) stretch position within the lane's group of 32
            tm.par([&](int lane) {
                int g0 = lane & ~31;
                uint32_t k = 0;
                int j = lane - 1;
                while (j >= g0 && s_a[j]) { ++k; --j; }
                s_b[lane] = k | (j < g0 ? 0x80000000u : 0u);    // high bit: the stretch reaches the group start
            });
            // (c) carry across groups of 32 (one thread; T/32 groups)
            tm.par([&](int lane) {
                if (lane != 0) return;
                uint32_t run = carry_run;
                for (int g = 0; g < T / 32; ++g) {
                    s_m[g] = run;
                    uint32_t last = s_b[g * 32 + 31];
                    uint32_t trail = s_a[g * 32 + 31] ? (last & 0x7FFFFFFFu) + 1u : 0u;
                    bool all = s_a[g * 32 + 31] && (last & 0x80000000u);   // 32 flags set
                    run = all ? run + 32u : trail;
                }
                s_m[T / 32] = run;
            });
            // (d) selection, survival, and the values to move
            uint32_t alive_total = 0;
            tm.par([&](int lane) {
                uint32_t kb = s_b[lane];
                uint32_t k = (kb & 0x7FFFFFFFu) + ((kb & 0x80000000u) ? s_m[lane >> 5] : 0u);
                uint32_t sel = (s_a[lane] && !(k & 1u)) ? 1u : 0u;
                s_c[lane] = sel;
            });
            tm.par([&](int lane) {
                uint32_t e = base + lane;
                uint32_t dead = lane ? s_c[lane - 1] : prev_sel;
                s_b[lane] = (e < n && !dead) ? 1u : 0u;        // alive
            });
            // values must be read before anything is overwritten
            tm.par([&](int lane) {
                uint32_t e = base + lane;
                if (e < n && s_b[lane]) {
                    uint32_t sel = s_c[lane];
                    tm.keep(lane, 0) = sel ? nw[e] : ids[e];
                    tm.keep(lane, 1) = sel ? kDirty : rk[e];
                    tm.keep(lane, 2) = nw[e];
                }
            });
            const uint32_t last_sel = s_c[T - 1];
            const uint32_t run_out = s_m[T / 32];
            // s_a is free now: reuse it for the scan of alive flags
            tm.par([&](int lane) { s_a[lane] = s_b[lane]; });
            tm.excl_scan(s_a, &alive_total);
            tm.par([&](int lane) {
                if (s_b[lane]) {
                    uint32_t d = out_base + s_a[lane];
                    ids[d] = tm.keep(lane, 0);
                    rk[d] = tm.keep(lane, 1);
                    nw[d] = tm.keep(lane, 2);
                }
            });
            out_base += alive_total;
            carry_run = run_out;
            prev_sel = last_sel;
        }
        n = out_base;
        // ---- re-probe the pairs next to a merge ----
        tm.par([&](int lane) {
            for (uint32_t p = lane; p < n; p += T) {
                bool d0 = rk[p] == kDirty, d1 = p + 1 < n && rk[p + 1] == kDirty;
                if (d0 || d1) nw[p] = kReprobe;
            }
        });
        tm.par([&](int lane) {
            for (uint32_t p = lane; p < n; p += T) {
                if (nw[p] != kReprobe) continue;
                if (p + 1 < n) { RankRes r = probe_rule(a.tb, ids[p], ids[p + 1]); rk[p] = r.rank; nw[p] = r.res; }
                else { rk[p] = kNoRank; nw[p] = 0; }
            }
        });
    }
    return n;
}

// End (exclusive, global byte position) of the pre-token starting at g, found by
// scanning the boundary bits; tiles without any boundary are skipped in one step.
// Where the pre-token that starts at g ends (the next boundary bit, or the end of the text), by the whole
// block: 256 mask words (8 KB of text) a step.  One thread going through the mask a word at a time took
// longer over a 36 KB pre-token than the block then took to merge it.  `scratch`: kThreads words.
template <class Blk>
GTOK_DEV uint32_t find_word_end(Blk& blk, const EncodeArgs& a, uint32_t* scratch, uint32_t g, uint32_t n) {
    const uint32_t n_words = ((n + kTile - 1) / kTile) * kTileWords;
    uint32_t wi = g >> 5;
    {
        uint32_t bits = ldg(a.bmask + wi) & ~((2u << (g & 31)) - 1u);
        if ((g & 31) == 31) bits = 0;
        if (bits) { const uint32_t e = wi * 32 + ffs32(bits); return e < n ? e : n; }
    }
    for (uint32_t base = wi + 1;; base += kThreads) {
        if (base >= n_words) return n;
        blk.par([&](int tid) {
            const uint32_t w = base + static_cast<uint32_t>(tid);
            scratch[tid] = (w >= n_words || ldg(a.bmask + w)) ? static_cast<uint32_t>(tid) : 0xFFFFFFFFu;
        });
        const uint32_t m = blk.reduce_min(scratch);
        if (m == 0xFFFFFFFFu) continue;
        const uint32_t w = base + m;
        if (w >= n_words) return n;
        const uint32_t e = w * 32 + ffs32(ldg(a.bmask + w));
        return e < n ? e : n;
    }
}

template <class Blk>
struct BlockTeam {
    static constexpr int kSize = kThreads;
    Blk& blk;
    uint32_t* keepbuf;   // [3 * kThreads] in shared memory
    GTOK_DEV BlockTeam(Blk& b, uint32_t* kb) : blk(b), keepbuf(kb) {}
    template <class F> GTOK_DEV void par(F f) { blk.par(f); }
    GTOK_DEV void excl_scan(uint32_t* arr, uint32_t* total) { blk.excl_scan(arr, total); }
    GTOK_DEV uint32_t reduce_min(uint32_t* arr) { return blk.reduce_min(arr); }
    GTOK_DEV uint32_t& keep(int lane, int k) { return keepbuf[k * kThreads + lane]; }
};

// ---- kernel 2: every pre-token of a tile against the whole-word table ----------------
// Known pre-tokens get their id at once; the others are appended to the global lists that
// the miss kernel works through.  The tile's slots go to `stage` (and the few ids that
// spill past the tile's end to `ovf`), so that nothing here waits on a merge loop.
template <class Blk>
GTOK_DEV void words_tile(Blk& blk, const EncodeArgs& a, WordsSmem& sm, int tile) {
    const uint32_t n = ldg(a.meta);
    const uint32_t t0 = static_cast<uint32_t>(tile) * kTile;
    const uint32_t n_tiles = (n + kTile - 1) / kTile;
    const uint32_t n_words = n_tiles * kTileWords;
    const DeviceTables& tb = a.tb;
    auto mark = [&](int slot) {
        if (!a.phase_clk) return;
        blk.par([&](int tid) {
            if (tid != 0) return;
            unsigned long long t = cycle_now();
            if (slot >= 0) add_cycles(a.phase_clk + slot, t - sm.clk_last);
            sm.clk_last = t;
        });
    };
    mark(-1);
    // ---- W0: stage text, bit masks, byte ids ----
    blk.par([&](int tid) {
        for (int c = tid; c < (kTile + 64) / 16; c += kThreads) {
            uint32_t p = t0 + c * 16;
            uint32_t* dst = reinterpret_cast<uint32_t*>(sm.txt + c * 16);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a.text + p);
#if defined(__CUDA_ARCH__)
            *reinterpret_cast<uint4*>(dst) = ld128(reinterpret_cast<const uint4*>(src));
#else
            for (int k = 0; k < 4; ++k) dst[k] = src[k];
#endif
        }
        for (int wd = tid; wd < kTileWords + 4; wd += kThreads) {
            uint32_t gw = tile * kTileWords + wd;
            sm.bm[wd] = gw < n_words ? ldg(a.bmask + gw) : 0u;
            sm.am[wd] = (tb.added_max_bytes && gw < n_words) ? ldg(a.amask + gw) : 0u;
        }
        sm.b2i[tid] = ldg(tb.byte_to_id + tid);
        for (int i = tid; i < kTile + kTokExtra; i += kThreads) sm.tok[i] = kInvalidTok;
        if (tid < 12) sm.ctr[tid] = 0;
    });
    mark(8);
    // ---- W1: the tile's pre-token starts as an ordered list ----
    blk.par([&](int tid) {
        uint32_t bits = (sm.bm[tid >> 1] >> ((tid & 1) * 16)) & 0xFFFFu;
        sm.scan[tid] = popc32(bits);
    });
    uint32_t n_starts = 0;
    blk.excl_scan(sm.scan, &n_starts);
    blk.par([&](int tid) {
        uint32_t bits = (sm.bm[tid >> 1] >> ((tid & 1) * 16)) & 0xFFFFu;
        uint32_t at = sm.scan[tid];
        while (bits) {
            int k = ffs32(bits);
            bits &= bits - 1;
            sm.wl[at++] = static_cast<uint16_t>(tid * kPer + k);
        }
        if (tid == 0) {
            // end of the last pre-token: the first boundary in the 64 staged bytes past the tile, if any
            uint32_t e = 0xFFFFu;
            if (sm.bm[kTileWords]) e = kTile + ffs32(sm.bm[kTileWords]);
            else if (sm.bm[kTileWords + 1]) e = kTile + 32 + ffs32(sm.bm[kTileWords + 1]);
            sm.wl[n_starts] = static_cast<uint16_t>(e);
        }
    });
    mark(9);
    // ---- W2: one table probe per pre-token, four in flight per thread ----
    blk.par([&](int tid) {
        uint32_t known = 0;                                  // ids this thread settles here
        for (uint32_t base = tid; base < n_starts; base += kThreads * 4) {
            uint32_t wo[4], wlen[4], wh[4];
            uint64_t wk0[4], wk1[4];
            bool wp[4];
#if defined(__CUDA_ARCH__)
            uint4 sa[4], sb[4];
#pragma unroll
#endif
            for (int u = 0; u < 4; ++u) {
                wp[u] = false;
                const uint32_t i = base + u * kThreads;
                if (i >= n_starts) continue;
                const uint32_t o = sm.wl[i], g = t0 + o;
                if (g >= n) continue;
                const uint32_t e = sm.wl[i + 1];
                uint32_t len = 0;                     // 0 = runs past the staged window
                if (e != 0xFFFFu) len = e - o;
                else if (t0 + kTile + 64 >= n) len = n - g;
                if (len && g + len > n) len = n - g;
                if ((sm.txt[o] & 0xC0u) == 0x80u && tb.family != 4u) continue;      // stray continuation bytes opening a document (the Gemma-3 shape spells every byte)
                if ((sm.am[o >> 5] >> (o & 31)) & 1u) {
                    sm.tok[o] = a.stage[g];                 // an added token: its id was left here when the literal was matched
                    ++known;
                    continue;
                }
                if (len == 0 || len > kMedWordMax) {
                    uint32_t slot = shared_add(&sm.ctr[C_NTEAM], 1u);
                    if (slot < kLongPerTile) { sm.lng_o[slot] = o; sm.lng_len[slot] = len; }
                    else global_or(a.ctl + CTL_ERR, kErrInternal);
                    continue;
                }
                if (len > kShortWordMax && !a.one_list) {
                    if (len > static_cast<uint32_t>(kMedSplit) && len <= static_cast<uint32_t>(kMedSplit1)) {
                        sm.med1[shared_add(&sm.ctr[C_NMED1], 1u)] = o | (len << 12);
                        continue;
                    }
                    const bool big = len > static_cast<uint32_t>(kMedSplit);
                    const uint32_t slot = shared_add(&sm.ctr[big ? C_NMED : C_NMED2], 1u);
                    sm.med[big ? slot : kTile / 16 - 1 - slot] = o | (len << 12);
                    continue;
                }
                if (len > kWordKeyMax) {
                    uint32_t slot = shared_add(&sm.ctr[C_NMISS], 1u);
                    sm.miss[slot] = o | (len << 12);
                    continue;
                }
                uint64_t k0 = 0, k1 = 0;
                for (uint32_t b = 0; b < len && b < 8; ++b) k0 |= static_cast<uint64_t>(sm.txt[o + b]) << (8 * b);
                for (uint32_t b = 8; b < len; ++b) k1 |= static_cast<uint64_t>(sm.txt[o + b]) << (8 * (b - 8));
                k1 |= static_cast<uint64_t>(len) << 56;
                wo[u] = o; wlen[u] = len; wk0[u] = k0; wk1[u] = k1;
                wh[u] = word_hash(k0, k1) & tb.word_mask;
                wp[u] = true;
#if defined(__CUDA_ARCH__)
                const uint4* sp = reinterpret_cast<const uint4*>(tb.word + wh[u]);
                sa[u] = __ldg(sp);
                sb[u] = __ldg(sp + 1);
#endif
            }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
            for (int u = 0; u < 4; ++u) {
                if (!wp[u]) continue;
                uint32_t id;
#if defined(__CUDA_ARCH__)
                const uint64_t s0 = (static_cast<uint64_t>(sa[u].y) << 32) | sa[u].x, s1 = (static_cast<uint64_t>(sa[u].w) << 32) | sa[u].z;
                if (sb[u].x == kNoToken) id = kNoToken;
                else if (s0 == wk0[u] && s1 == wk1[u]) id = sb[u].x;
                else id = probe_word_from(tb, wk0[u], wk1[u], (wh[u] + 1u) & tb.word_mask);     // the home slot holds another key: walk on from the next
#else
                id = probe_word(tb, wk0[u], wk1[u]);
#endif
                const uint32_t o = wo[u], len = wlen[u];
                if (id != kNoToken) { sm.tok[o] = id; ++known; continue; }
                if (len == 1) { sm.tok[o] = sm.b2i[sm.txt[o]]; ++known; continue; }
                uint32_t slot = shared_add(&sm.ctr[C_NMISS], 1u);
                sm.miss[slot] = o | (len << 12);
            }
        }
        if (known) shared_add(&sm.ctr[C_NKNOWN], known);
    });
    mark(10);
    // ---- W3: hand the unknown and the long pre-tokens to the global lists; write the slots out ----
    blk.par([&](int tid) {
        if (tid != 0) return;
        uint32_t nm = sm.ctr[C_NMISS], nl = sm.ctr[C_NTEAM];
        if (nl > kLongPerTile) nl = kLongPerTile;
        sm.ctr[C_NTEAM] = nl;
        const uint32_t nd = sm.ctr[C_NMED], nd2 = sm.ctr[C_NMED2], nd1 = sm.ctr[C_NMED1];
        a.tile_tok[tile] = sm.ctr[C_NKNOWN];            // the merge kernel adds what it settles
#if defined(__CUDA_ARCH__)
        sm.ctr[C_BASEM] = nm ? atomicAdd(a.ctl + CTL_NMISS, nm) : 0u;
        sm.ctr[C_BASEL] = nl ? atomicAdd(a.ctl + CTL_NLONG, nl) : 0u;
        sm.ctr[C_BASED] = nd ? atomicAdd(a.ctl + CTL_NMED, nd) : 0u;
        sm.ctr[C_BASED2] = nd2 ? atomicAdd(a.ctl + CTL_NMED2, nd2) : 0u;
        sm.ctr[C_BASED1] = nd1 ? atomicAdd(a.ctl + CTL_NMED1, nd1) : 0u;
#else
        sm.ctr[C_BASEM] = a.ctl[CTL_NMISS]; a.ctl[CTL_NMISS] += nm;
        sm.ctr[C_BASEL] = a.ctl[CTL_NLONG]; a.ctl[CTL_NLONG] += nl;
        sm.ctr[C_BASED] = a.ctl[CTL_NMED]; a.ctl[CTL_NMED] += nd;
        sm.ctr[C_BASED2] = a.ctl[CTL_NMED2]; a.ctl[CTL_NMED2] += nd2;
        sm.ctr[C_BASED1] = a.ctl[CTL_NMED1]; a.ctl[CTL_NMED1] += nd1;
#endif
    });
    {
        const uint32_t nm = sm.ctr[C_NMISS], nl = sm.ctr[C_NTEAM], bm0 = sm.ctr[C_BASEM], bl0 = sm.ctr[C_BASEL];
        const uint32_t nd = sm.ctr[C_NMED], bd0 = sm.ctr[C_BASED], nd2 = sm.ctr[C_NMED2], bd2 = sm.ctr[C_BASED2];
        const uint32_t nd1 = sm.ctr[C_NMED1], bd1 = sm.ctr[C_BASED1];
        blk.par([&](int tid) {
            for (uint32_t i = tid; i < nm; i += kThreads) {
                uint32_t mv = sm.miss[i];
                a.gmiss[bm0 + i] = static_cast<unsigned long long>(t0 + (mv & 0xFFFu)) | (static_cast<unsigned long long>(mv >> 12) << 32);
            }
            for (uint32_t i = tid; i < nd; i += kThreads) {
                uint32_t mv = sm.med[i];
                a.gmed[bd0 + i] = static_cast<unsigned long long>(t0 + (mv & 0xFFFu)) | (static_cast<unsigned long long>(mv >> 12) << 32);
            }
            for (uint32_t i = tid; i < nd1; i += kThreads) {
                uint32_t mv = sm.med1[i];
                a.gmed1[bd1 + i] = static_cast<unsigned long long>(t0 + (mv & 0xFFFu)) | (static_cast<unsigned long long>(mv >> 12) << 32);
            }
            for (uint32_t i = tid; i < nd2; i += kThreads) {
                uint32_t mv = sm.med[kTile / 16 - 1 - i];
                a.gmed[a.gmed_cap - 1 - (bd2 + i)] = static_cast<unsigned long long>(t0 + (mv & 0xFFFu)) | (static_cast<unsigned long long>(mv >> 12) << 32);
            }
            for (uint32_t i = tid; i < nl; i += kThreads) {
                a.glong_g[bl0 + i] = t0 + sm.lng_o[i];
                a.glong_len[bl0 + i] = sm.lng_len[i];
                a.glong_cnt[bl0 + i] = 0;
                sm.tok[sm.lng_o[i]] = kLongRef | (bl0 + i);
            }
        });
        blk.par([&](int tid) {
#if defined(__CUDA_ARCH__)
            for (int c = tid; c < kTile / 4; c += kThreads)
                reinterpret_cast<uint4*>(a.stage + t0)[c] = reinterpret_cast<const uint4*>(sm.tok)[c];
#else
            for (int i = tid; i < kTile; i += kThreads) a.stage[t0 + i] = sm.tok[i];
#endif
            if (tid < kTokExtra) a.ovf[static_cast<size_t>(tile) * kTokExtra + tid] = sm.tok[kTile + tid];
        });
    }
    mark(11);
}

// Stores the k-th id of the pre-token that starts at byte g.
GTOK_DEV void put_id(const EncodeArgs& a, uint32_t g, uint32_t k, uint32_t id) {
    const uint32_t tile = g / kTile, t1 = (tile + 1) * kTile;
    if (g + k < t1) a.stage[g + k] = id;
    else a.ovf[static_cast<size_t>(tile) * kTokExtra + (g + k - t1)] = id;
}

// The first two phases of a batch over the block's arena (sm.word holds the batch's entries, position |
// length << 32, 0 = none): all threads fetch the bytes, a slot each, so that the loads overlap ...
constexpr uint32_t kPendingRank = 0xFFFFFFFDu;
template <class Blk>
GTOK_DEV void arena_fill(Blk& blk, const EncodeArgs& a, MissSmem& sm, uint32_t* ids, uint32_t* rk, uint32_t batch, uint32_t max_len) {
    const uint32_t slots = batch * max_len;
    blk.par([&](int tid) {
        for (uint32_t x = tid; x < slots; x += kThreads) {
            const uint32_t w = (x >> 2) % batch, r = ((x >> 2) / batch) * 4u + (x & 3u);
            const unsigned long long wv = sm.word[w];
            const uint32_t g = static_cast<uint32_t>(wv), len = static_cast<uint32_t>(wv >> 32);
            if (r >= ((len + 3u) & ~3u)) continue;                  // beyond the pre-token's last group: never read
            if (r >= len) { rk[x] = kNoRank; continue; }            // padding of the last group
            const uint32_t bt = ldg(a.text + g + r);
            sm.rawb[w * max_len + r] = static_cast<uint8_t>(bt);
            ids[x] = sm.b2i[bt];
            rk[x] = (r + 1 < len) ? kPendingRank : kNoRank;
            sm.lnk[x] = static_cast<uint16_t>(((r ? r - 1 : 0xFFu) << 8) | (r + 1 < len ? r + 1 : 0xFFu));
        }
    });
}
// ... and probe all adjacent pairs, a slot each; then the lowest key of every group of four slots
// (pre-tokens of more than 16 bytes search through these).
template <class Blk>
GTOK_DEV void arena_pairs(Blk& blk, const EncodeArgs& a, MissSmem& sm, uint32_t* ids, uint32_t* rk, uint32_t* nw, uint32_t batch, uint32_t max_len) {
    const uint32_t slots = batch * max_len, stride = batch * 4u;
    blk.par([&](int tid) {
        for (uint32_t x = tid; x < slots; x += kThreads) {
            const uint32_t w = (x >> 2) % batch, r = ((x >> 2) / batch) * 4u + (x & 3u);
            const uint32_t len = static_cast<uint32_t>(sm.word[w] >> 32);
            if (r + 1 >= len || rk[x] != kPendingRank) continue;
            RankRes q = probe_rule(a.tb, ids[x], ids[arena_at(4u * w, stride, r + 1)]);
            rk[x] = rank_key(q.rank, r);
            nw[x] = q.res;
        }
    });
    if (max_len > 16u) {
        blk.par([&](int tid) {
            for (uint32_t i = tid; i < slots / 4u; i += kThreads) {
                const uint32_t w = (i >> 2) % batch, g = ((i >> 2) / batch) * 4u + (i & 3u);
                const uint32_t len = static_cast<uint32_t>(sm.word[w] >> 32);
                uint32_t m = kNoRank;
                if (g * 4u < len) for (uint32_t r = g * 4u; r < g * 4u + 4u; ++r) { const uint32_t v = rk[arena_at(4u * w, stride, r)]; if (v < m) m = v; }
                sm.gmin[i] = m;
            }
        });
    }
}

// ---- kernel 3a: one batch of unknown pre-tokens (2..64 bytes), one per thread ----------
// All threads fetch the batch's bytes into the block's arena and probe the initial pairs, a
// slot each; then the thread that owns a pre-token merges it (lowest rank first) and stores
// the ids.  `max_len` is the longest pre-token of the batch's length class: batch * max_len
// slots fit the arena.
// kMode 1 (`share`): a call with take > batch hands back what it cannot merge in one arena; kMode 2
// (`surplus`): the entries are such handed-back ones.  (Template values, so that the plain call's code is
// what it was without them.)
template <class Blk, int kMode = 0>
GTOK_DEV void miss_batch(Blk& blk, const EncodeArgs& a, MissSmem& sm, const unsigned long long* list, int dir, uint32_t first, uint32_t n_miss,
                         uint32_t batch, uint32_t max_len, uint32_t take) {
    constexpr bool share = kMode == 1, surplus = kMode == 2;
    const DeviceTables& tb = a.tb;
    uint32_t* ids = sm.ws;
    uint32_t* rk = sm.ws + kArenaSyms;
    uint32_t* nw = sm.ws + 2 * kArenaSyms;
    // `take` list entries belong to this call.  take > batch: most entries are expected to be vocabulary
    // tokens as they stand (ignore_merges), so every thread first looks one entry up as a whole, straight
    // from the text, and only what is left enters the arena, `batch` pre-tokens at a time.
    const uint32_t n_take = n_miss - first < take ? n_miss - first : take;
    const bool filtered = take > batch;
    const uint32_t stride = batch * 4u;                 // arena elements from one group of a pre-token to its next
    auto mark = [&](int slot) {
        if (!a.phase_clk) return;
        blk.par([&](int tid) {
            if (tid != 0) return;
            unsigned long long t = cycle_now();
            if (slot >= 0) add_cycles(a.phase_clk + slot, t - sm.clk_last);
            sm.clk_last = t;
#if defined(__CUDA_ARCH__)
            // timeline table 4, row of this block: when each phase of its (last) batch ended, and which class that was
            if (blockIdx.x < kTlBlocks) {
                unsigned long long ns;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
                unsigned long long* row = a.phase_clk + kPhaseWords + (static_cast<size_t>(4) * kTlBlocks + blockIdx.x) * kTlSlots;
                row[slot < 0 ? 0 : slot - 15] = ns;                 // slots 16..20 -> 1..5
                row[7] = max_len * 1000ull + n_take;
            }
#endif
        });
    };
    mark(-1);
    uint32_t n_cand = n_take;
    if (filtered) {
        // the entries' bytes into shared memory first (all threads, a byte each, so the loads overlap):
        // max_len bytes apart in the arena, which nothing uses yet
        uint8_t* stage_bytes = reinterpret_cast<uint8_t*>(sm.ws);
        blk.par([&](int tid) {
            if (tid == 0) sm.ctr[C_USED] = 0;
            if (static_cast<uint32_t>(tid) < n_take) sm.cand[tid] = list[static_cast<long long>(dir) * static_cast<long long>(first + tid)];
        });
        blk.par([&](int tid) {
            // (a word of four bytes per load where the address allows, and four loads in flight per thread:
            // a plain byte loop waits for every byte in turn, thirty-two memory round trips in a row)
            const uint32_t words_per = max_len / 4u;
            for (uint32_t x0 = tid; x0 < n_take * words_per; x0 += 4 * kThreads) {
                uint32_t v[4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
                for (int u = 0; u < 4; ++u) {
                    const uint32_t x = x0 + u * kThreads;
                    v[u] = 0;
                    if (x >= n_take * words_per) continue;
                    const uint32_t w = x / words_per, r = (x % words_per) * 4u;
                    const unsigned long long wv = sm.cand[w];
                    const uint32_t g = static_cast<uint32_t>(wv), len = static_cast<uint32_t>(wv >> 32);
                    if (r >= len) continue;
                    const uint8_t* p = a.text + g + r;
                    if (r + 4u <= len && (reinterpret_cast<uintptr_t>(p) & 3u) == 0) v[u] = ldg(reinterpret_cast<const uint32_t*>(p));
                    else for (uint32_t b = 0; b < 4u && r + b < len; ++b) v[u] |= static_cast<uint32_t>(ldg(p + b)) << (8 * b);
                }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
                for (int u = 0; u < 4; ++u) {
                    const uint32_t x = x0 + u * kThreads;
                    if (x < n_take * words_per) reinterpret_cast<uint32_t*>(stage_bytes)[x] = v[u];     // bytes past the entry's end are never read
                }
            }
        });
        typename Blk::template Local<unsigned long long> left;
        blk.par([&](int tid) {
            left.at(tid) = 0ull;
            if (static_cast<uint32_t>(tid) >= n_take) return;
            const unsigned long long wv = sm.cand[tid];
            const uint32_t g = static_cast<uint32_t>(wv), len = static_cast<uint32_t>(wv >> 32);
            const uint32_t id = probe_long_bytes(tb, stage_bytes + tid * max_len, len);
            if (id != kNoToken) { put_id(a, g, 0, id); global_add(a.tile_tok + g / kTile, 1u); }
            else left.at(tid) = wv;
        });
        blk.par([&](int tid) {
            const unsigned long long wv = left.at(tid);
            if (wv) sm.cand[shared_add(&sm.ctr[C_USED], 1u)] = wv;
        });
        n_cand = sm.ctr[C_USED];
        if (share) {
            // What does not fit one arena goes back to the head of this call's stretch of the list, its
            // count in front of it, for whichever block is free first (miss_surplus): a text whose long
            // pre-tokens are not in the vocabulary would otherwise keep this block for three arenas in a row.
            const uint32_t extra = n_cand > batch ? n_cand - batch : 0u;
            unsigned long long* wlist = const_cast<unsigned long long*>(list);
            blk.par([&](int tid) {
                if (tid == 0) store_state(wlist + static_cast<long long>(dir) * static_cast<long long>(first), extra);
                if (static_cast<uint32_t>(tid) < extra)
                    store_state(wlist + static_cast<long long>(dir) * static_cast<long long>(first + 1u + tid), sm.cand[batch + tid]);
            });
            blk.par([&](int tid) {
                if (tid != 0) return;
                if (extra) global_add(a.ctl + CTL_NSURPLUS, extra);
                release_add(a.ctl + CTL_FILTERED, 1u);
            });
            if (n_cand > batch) n_cand = batch;
        }
    }
    for (uint32_t done = 0; done < n_cand; done += batch) {
    const uint32_t n_here = n_cand - done < batch ? n_cand - done : batch;
    blk.par([&](int tid) {
        if (static_cast<uint32_t>(tid) < batch)
            sm.word[tid] = static_cast<uint32_t>(tid) >= n_here ? 0ull : filtered ? sm.cand[done + tid]
                           : surplus ? load_state(list + static_cast<long long>(dir) * static_cast<long long>(first + tid))   // written by another block
                           : list[static_cast<long long>(dir) * static_cast<long long>(first + tid)];   // dir = -1: a list that grows downwards
    });
    mark(16);
    arena_fill(blk, a, sm, ids, rk, batch, max_len);
    mark(17);
    // owner: a pre-token of 16 bytes or more that is itself in the vocabulary (ignore_merges)
    if (!filtered && !surplus && tb.ignore_merges && max_len > static_cast<uint32_t>(kWordKeyMax)) {
        blk.par([&](int tid) {
            if (static_cast<uint32_t>(tid) >= n_here) return;
            const unsigned long long wv = sm.word[tid];
            const uint32_t g = static_cast<uint32_t>(wv), len = static_cast<uint32_t>(wv >> 32);
            if (len <= kWordKeyMax) return;
            uint32_t id = probe_long_bytes(tb, sm.rawb + tid * max_len, len);
            if (id == kNoToken) return;
            put_id(a, g, 0, id);
            global_add(a.tile_tok + g / kTile, 1u);
            sm.word[tid] = 0ull;                                    // done
        });
    }
    mark(18);
    arena_pairs(blk, a, sm, ids, rk, nw, batch, max_len);
    mark(19);
    blk.par([&](int tid) {
        if (static_cast<uint32_t>(tid) >= n_here) return;
        const unsigned long long wv = sm.word[tid];
        const uint32_t g = static_cast<uint32_t>(wv), len = static_cast<uint32_t>(wv >> 32);
        if (len == 0) return;
        const uint32_t cnt = bpe_arena(a, ids, rk, nw, sm.lnk, sm.gmin, 4u * tid, stride, len, [&](uint32_t k, uint32_t id) { put_id(a, g, k, id); });
        global_add(a.tile_tok + g / kTile, cnt);
    });
    mark(20);
    }
}

// The two rare modes as functions of their own: inlined into the kernel beside the plain call they cost
// every text a few percent of the kernel (registers and code size), used or not.
template <class Blk>
GTOK_DEV_NOINLINE void miss_batch_sharing(Blk& blk, const EncodeArgs& a, MissSmem& sm, const unsigned long long* list, int dir, uint32_t first, uint32_t n_miss,
                                          uint32_t batch, uint32_t max_len, uint32_t take) {
    miss_batch<Blk, 1>(blk, a, sm, list, dir, first, n_miss, batch, max_len, take);
}
template <class Blk>
GTOK_DEV_NOINLINE void miss_batch_surplus(Blk& blk, const EncodeArgs& a, MissSmem& sm, const unsigned long long* list, int dir, uint32_t first, uint32_t n_miss) {
    miss_batch<Blk, 2>(blk, a, sm, list, dir, first, n_miss, kMedBatchB, kMedSplit, kMedBatchB);
}

// What a call of the 17..32-byte class with `share` left behind: chunk `chunk` of the surplus of the
// call that began at list entry `first`.  The entries are known not to be vocabulary tokens.
constexpr uint32_t kSurplusChunks = (kMedTakeB - kMedBatchB + kMedBatchB - 1) / kMedBatchB;
template <class Blk>
GTOK_DEV void miss_surplus(Blk& blk, const EncodeArgs& a, MissSmem& sm, const unsigned long long* list, int dir, uint32_t first, uint32_t chunk) {
    const uint32_t extra = static_cast<uint32_t>(load_state(list + static_cast<long long>(dir) * static_cast<long long>(first)));
    if (chunk * kMedBatchB >= extra) return;
    miss_batch_surplus(blk, a, sm, list, dir, first + 1u + chunk * kMedBatchB, first + 1u + extra);
}

// ---- run-length path for long pre-tokens made of a few byte runs ------------------------
// A very long pre-token is, in practice, a run of one character (spaces, newlines, dashes,
// '=' ...) or a few such runs.  Its symbol sequence is kept as (symbol, count) runs and a
// round applies every occurrence of the lowest-rank pair at once: inside a run s^k the
// pair (s, s) merges into t^(k/2) plus a left-over s, leftmost pairs first, and a pair
// (l, r) across two runs takes one symbol from each.  For a vocabulary with monotone ranks
// this is what the greedy loop does, one merge at a time (same argument as in team_bpe).
// The number of runs stays tiny, so a round is one parallel batch of probes plus a few
// hundred instructions by one thread, instead of passes over tens of thousands of symbols.
// Returns false (nothing written) when the pre-token has too many runs, now or later.
constexpr int kRleMax = 64;

template <class Blk>
GTOK_DEV bool rle_word(Blk& blk, const EncodeArgs& a, MissSmem& sm, uint32_t li, uint32_t g, uint32_t len) {
    uint32_t* w = sm.ws;
    uint32_t* s_cnt = w;                      // [kThreads] scan scratch
    uint32_t* sym = w + kThreads;             // run symbols, counts, and their rebuilt copies
    uint32_t* cnt = sym + (kRleMax + 2);
    uint32_t* sym2 = cnt + (kRleMax + 2);
    uint32_t* cnt2 = sym2 + (kRleMax + 2);
    uint32_t* r_self = cnt2 + (kRleMax + 2);  // rank / result of (s_i, s_i) and of (s_i, s_i+1)
    uint32_t* t_self = r_self + (kRleMax + 2);
    uint32_t* r_next = t_self + (kRleMax + 2);
    uint32_t* t_next = r_next + (kRleMax + 2);
    uint32_t* offs = t_next + (kRleMax + 2);
    // Each thread takes a stretch of whole 16-byte lines of the text (the first and the last thread also the ragged ends).
    // ---- byte runs ----
    // A line whose sixteen bytes all equal the byte before it opens no run: such lines, nearly all of a
    // long run, cost one 128-bit load and a few compares; the others are looked at byte by byte.
    uint32_t head = (16u - (g & 15u)) & 15u;                          // bytes before the first whole line
    if (head > len) head = len;
    const uint32_t lines = (len - head) / 16u;
    const uint32_t per = (lines + kThreads - 1) / kThreads;            // lines per thread
    auto scan_stretch = [&](int tid, auto&& on_start) {
        // thread t: lines [t * per, (t + 1) * per) of the pre-token; thread 0 also the head, the last thread the tail
        const uint32_t l0 = static_cast<uint32_t>(tid) * per < lines ? static_cast<uint32_t>(tid) * per : lines;
        const uint32_t l1 = (static_cast<uint32_t>(tid) + 1u) * per < lines ? (static_cast<uint32_t>(tid) + 1u) * per : lines;
        const uint32_t lo = tid == 0 ? 0u : head + 16u * l0;
        const uint32_t hi = tid == kThreads - 1 ? len : head + 16u * l1;
        uint32_t i = lo;
        uint32_t prev = i ? ldg(a.text + g + i - 1) : 0x100u;
        while (i < hi) {
            if (((g + i) & 15u) == 0 && i + 16u <= hi && prev < 0x100u) {
                const uint32_t* p4 = reinterpret_cast<const uint32_t*>(a.text + g + i);
                const uint32_t pat = prev * 0x01010101u;
                if (ldg(p4) == pat && ldg(p4 + 1) == pat && ldg(p4 + 2) == pat && ldg(p4 + 3) == pat) { i += 16u; continue; }
            }
            const uint32_t b = ldg(a.text + g + i);
            if (b != prev) on_start(i, b);
            prev = b;
            ++i;
        }
    };
    blk.par([&](int tid) {
        uint32_t c = 0;
        scan_stretch(tid, [&](uint32_t, uint32_t) { ++c; });
        s_cnt[tid] = c;
    });
    uint32_t n_runs = 0;
    blk.excl_scan(s_cnt, &n_runs);
    if (n_runs > static_cast<uint32_t>(kRleMax)) return false;
    blk.par([&](int tid) {
        uint32_t at = s_cnt[tid];
        scan_stretch(tid, [&](uint32_t i, uint32_t b) { sym[at] = sm.b2i[b]; offs[at] = i; ++at; });
    });
    blk.par([&](int tid) {
        if (static_cast<uint32_t>(tid) < n_runs) cnt[tid] = (static_cast<uint32_t>(tid) + 1 < n_runs ? offs[tid + 1] : len) - offs[tid];
        if (tid == 0) { sm.ctr[C_TMP] = n_runs; sm.ctr[C_TMP2] = 0; }
    });
    // ---- rounds ----
    for (;;) {
        const uint32_t R = sm.ctr[C_TMP];
        blk.par([&](int tid) {
            const uint32_t i = static_cast<uint32_t>(tid) >> 1;
            if (i >= R) return;
            if (!(tid & 1)) {
                RankRes q{kNoRank, 0};
                if (cnt[i] >= 2) q = probe_rule(a.tb, sym[i], sym[i]);
                r_self[i] = q.rank; t_self[i] = q.res;
            } else {
                RankRes q{kNoRank, 0};
                if (i + 1 < R) q = probe_rule(a.tb, sym[i], sym[i + 1]);
                r_next[i] = q.rank; t_next[i] = q.res;
            }
        });
        blk.par([&](int tid) {
            if (tid != 0) return;
            uint32_t m = kNoRank, l = 0, r = 0, t = 0;
            for (uint32_t i = 0; i < R; ++i) {
                if (r_self[i] < m) { m = r_self[i]; l = r = sym[i]; t = t_self[i]; }
                if (r_next[i] < m) { m = r_next[i]; l = sym[i]; r = sym[i + 1]; t = t_next[i]; }
            }
            if (m == kNoRank) { sm.ctr[C_TMP2] = 1; return; }            // finished
            uint32_t R2 = 0;
            bool over = false;
            auto emit = [&](uint32_t s, uint32_t c) {
                if (c == 0) return;
                if (R2 && sym2[R2 - 1] == s) { cnt2[R2 - 1] += c; return; }
                if (R2 >= static_cast<uint32_t>(kRleMax)) { over = true; return; }
                sym2[R2] = s; cnt2[R2] = c; ++R2;
            };
            for (uint32_t i = 0; i < R; ++i) {
                const uint32_t s = sym[i], c = cnt[i];
                if (l == r) {
                    if (s == l && c >= 2) { emit(t, c >> 1); emit(l, c & 1u); }
                    else emit(s, c);
                } else if (s == l && i + 1 < R && sym[i + 1] == r && c >= 1 && cnt[i + 1] >= 1) {
                    emit(l, c - 1); emit(t, 1); cnt[i + 1] -= 1;
                } else emit(s, c);
            }
            if (over) { sm.ctr[C_TMP2] = 2; return; }
            for (uint32_t i = 0; i < R2; ++i) { sym[i] = sym2[i]; cnt[i] = cnt2[i]; }
            sm.ctr[C_TMP] = R2;
        });
        const uint32_t state = sm.ctr[C_TMP2];
        if (state == 2) return false;
        if (state == 1) break;
    }
    // ---- expand the runs into ids ----
    const uint32_t R = sm.ctr[C_TMP];
    blk.par([&](int tid) {
        if (tid != 0) return;
        uint32_t acc = 0;
        for (uint32_t i = 0; i < R; ++i) { offs[i] = acc; acc += cnt[i]; }
        a.glong_cnt[li] = acc;
        global_add(a.tile_tok + g / kTile, acc);
    });
    blk.par([&](int tid) {
        for (uint32_t i = 0; i < R; ++i) {
            const uint32_t s = sym[i], c = cnt[i], o = g + offs[i];
            for (uint32_t k = tid; k < c; k += kThreads) a.gstage[o + k] = s;
        }
    });
    return true;
}

// ---- kernel 3b: one pre-token longer than 64 bytes, by the whole block ------------------
// ---- long pre-tokens in pieces ---------------------------------------------------------------
// A pre-token of thousands of symbols that is no handful of runs is cut into pieces of at most 64 bytes
// that are merged like ordinary unknown pre-tokens, a thread each, 48 to a batch -- instead of rounds over
// all of its symbols, one round per rank that occurs.  What makes that exact: with a monotone vocabulary
// the greedy loop applies its merges in order of rank, so a cut is a token boundary of the whole pre-token
// if and only if the pair across it never gets its turn: at every moment, the rule joining the symbol left
// of the cut to the symbol right of it (if there is one) has a rank at or above the rank at which the left
// symbol next merges leftwards, or above the rank at which the right symbol next merges rightwards.  Both
// symbols' histories come out of merging the two pieces independently (each piece's two edges are recorded
// as it is merged), and if every cut passes, the pieces' ids one after the other are the pre-token's ids.
//   pass 0   windows of 64 bytes around every 40th byte are merged; the token boundary nearest the middle
//            of each (at most 12 bytes away) becomes a cut -- a true boundary almost always, far from the
//            window's own ends as it is
//   pass 1   the pieces between the cuts are merged, ids and edge histories to the pre-token's workspace
//   check    every cut, a thread each; a cut that fails, a piece that comes out too long, a history that
//            outgrows its room: nothing has been written that matters, the caller takes the general path
//   commit   piece totals summed, ids moved together, counts published
// Workspace (the three per-byte arrays of the pre-token, relative to its start): gwork_rk holds the cuts and,
// behind them, 32 words per piece {id count, changes of the first symbol, changes of the last symbol, then up
// to seven (id, rank) pairs for each}; gwork_nw holds piece k's ids at its own bytes; gstage the result.
constexpr uint32_t kPieceStep = 40, kPieceHalf = 32, kPieceDev = 12, kPieceMax = 64, kPieceHist = 7, kPieceRec = 32;
constexpr uint32_t kPieceMinLen = 256;         // shorter long pre-tokens stay with the general path

struct PieceHistory {
    uint32_t* rec;          // the piece's 32-word record
    GTOK_DEV void first(uint32_t id, uint32_t rank) {
        const uint32_t k = rec[1];
        if (k < kPieceHist) { rec[3 + 2 * k] = id; rec[4 + 2 * k] = rank; }
        rec[1] = k + 1;
    }
    GTOK_DEV void last(uint32_t id, uint32_t rank) {
        const uint32_t k = rec[2];
        if (k < kPieceHist) { rec[3 + 2 * kPieceHist + 2 * k] = id; rec[4 + 2 * kPieceHist + 2 * k] = rank; }
        rec[2] = k + 1;
    }
};

template <class Blk>
GTOK_DEV bool pieces_word(Blk& blk, const EncodeArgs& a, MissSmem& sm, uint32_t li, uint32_t g, uint32_t len) {
    const DeviceTables& tb = a.tb;
    // cuts 1..K at about every kPieceStep bytes; cut 0 = 0, cut K + 1 = len
    const uint32_t K = (len - 12u) / kPieceStep;                      // the last piece stays within kPieceMax however its cut falls
    uint32_t* cuts = a.gwork_rk + g;
    const uint32_t rec0 = (K + 2u + 3u) & ~3u;
    if (rec0 + (K + 1u) * kPieceRec > len) return false;              // (only for pre-tokens far shorter than kPieceMinLen)
    uint32_t* recs = a.gwork_rk + g + rec0;
    uint32_t* piece_ids = a.gwork_nw + g;
    uint32_t* ids = sm.ws;
    uint32_t* rk = sm.ws + kArenaSyms;
    uint32_t* nw = sm.ws + 2 * kArenaSyms;
    constexpr uint32_t batch = kMedBatchA, max_len = kMedWordMax, stride = batch * 4u;
    static_assert(kPieceMax <= static_cast<uint32_t>(kMedWordMax) && 2 * kPieceHalf <= kPieceMax, "a piece is one arena pre-token");
    blk.par([&](int tid) { if (tid == 0) { sm.ctr[C_TMP2] = 0; cuts[0] = 0; cuts[K + 1] = len; } });
    // ---- pass 0: a cut near every kPieceStep-th byte ----
    for (uint32_t first = 0; first < K; first += batch) {
        const uint32_t n_here = K - first < batch ? K - first : batch;
        blk.par([&](int tid) {
            if (static_cast<uint32_t>(tid) >= batch) return;
            unsigned long long wv = 0ull;
            if (static_cast<uint32_t>(tid) < n_here) {
                const uint32_t c = kPieceStep * (first + tid + 1u);
                const uint32_t lo = c - kPieceHalf, hi = c + kPieceHalf < len ? c + kPieceHalf : len;      // c >= kPieceStep > kPieceHalf
                wv = static_cast<unsigned long long>(g + lo) | (static_cast<unsigned long long>(hi - lo) << 32);
            }
            sm.word[tid] = wv;
        });
        arena_fill(blk, a, sm, ids, rk, batch, max_len);
        arena_pairs(blk, a, sm, ids, rk, nw, batch, max_len);
        blk.par([&](int tid) {
            if (static_cast<uint32_t>(tid) >= n_here) return;
            const uint32_t wlen = static_cast<uint32_t>(sm.word[tid] >> 32);
            bpe_arena(a, ids, rk, nw, sm.lnk, sm.gmin, 4u * tid, stride, wlen, [](uint32_t, uint32_t) {});
            // the symbols left are the window's tokens; their first slots are the byte offsets where tokens begin
            uint32_t best = 0, best_dev = 0xFFFFFFFFu;
            for (uint32_t i = sm.lnk[arena_at(4u * tid, stride, 0)] & 0xFFu; i != 0xFFu; i = sm.lnk[arena_at(4u * tid, stride, i)] & 0xFFu) {
                const uint32_t dev = i > kPieceHalf ? i - kPieceHalf : kPieceHalf - i;
                if (dev < best_dev) { best_dev = dev; best = i; }
            }
            if (best_dev > kPieceDev) { sm.ctr[C_TMP2] = 1; return; }
            cuts[first + tid + 1u] = kPieceStep * (first + tid + 1u) - kPieceHalf + best;
        });
        if (sm.ctr[C_TMP2]) return false;
    }
    // ---- pass 1: the pieces ----
    for (uint32_t first = 0; first <= K; first += batch) {
        const uint32_t n_here = K + 1u - first < batch ? K + 1u - first : batch;
        blk.par([&](int tid) {
            if (static_cast<uint32_t>(tid) >= batch) return;
            unsigned long long wv = 0ull;
            if (static_cast<uint32_t>(tid) < n_here) {
                const uint32_t lo = cuts[first + tid], hi = cuts[first + tid + 1u];
                if (hi <= lo || hi - lo > kPieceMax) sm.ctr[C_TMP2] = 1;
                else wv = static_cast<unsigned long long>(g + lo) | (static_cast<unsigned long long>(hi - lo) << 32);
            }
            sm.word[tid] = wv;
        });
        if (sm.ctr[C_TMP2]) return false;
        arena_fill(blk, a, sm, ids, rk, batch, max_len);
        arena_pairs(blk, a, sm, ids, rk, nw, batch, max_len);
        blk.par([&](int tid) {
            if (static_cast<uint32_t>(tid) >= n_here) return;
            const unsigned long long wv = sm.word[tid];
            const uint32_t lo = static_cast<uint32_t>(wv) - g, plen = static_cast<uint32_t>(wv >> 32);
            uint32_t* rec = recs + static_cast<size_t>(first + tid) * kPieceRec;
            rec[1] = 0; rec[2] = 0;
            PieceHistory hist{rec};
            rec[0] = bpe_arena(a, ids, rk, nw, sm.lnk, sm.gmin, 4u * tid, stride, plen, [&](uint32_t k, uint32_t id) { piece_ids[lo + k] = id; }, hist);
            if (rec[1] > kPieceHist || rec[2] > kPieceHist) sm.ctr[C_TMP2] = 1;
        });
        if (sm.ctr[C_TMP2]) return false;
    }
    // ---- check every cut ----
    blk.par([&](int tid) {
        for (uint32_t k = 1u + tid; k <= K; k += kThreads) {
            const uint32_t* L = recs + static_cast<size_t>(k - 1u) * kPieceRec;      // the piece left of cut k: its last symbol
            const uint32_t* R = recs + static_cast<size_t>(k) * kPieceRec;           // the piece right of it: its first symbol
            const uint32_t nl = L[2], nr = R[1];
            uint32_t sl = sm.b2i[ldg(a.text + g + cuts[k] - 1u)], sr = sm.b2i[ldg(a.text + g + cuts[k])];
            uint32_t i = 0, j = 0;
            for (;;) {
                const uint32_t tl = i < nl ? L[4 + 2 * kPieceHist + 2 * i] : 0xFFFFFFFFu;      // rank at which the left symbol next changes
                const uint32_t tr = j < nr ? R[4 + 2 * j] : 0xFFFFFFFFu;
                const RankRes q = probe_rule(tb, sl, sr);
                if (q.rank != kNoRank && q.rank < tl && q.rank <= tr) { sm.ctr[C_TMP2] = 1; break; }   // the pair across the cut would merge
                if (i >= nl && j >= nr) break;
                // the side that changes first (on equal ranks the left one: its pair lies further left)
                if (tl <= tr) { sl = L[3 + 2 * kPieceHist + 2 * i]; ++i; }
                else { sr = R[3 + 2 * j]; ++j; }
            }
        }
    });
    if (sm.ctr[C_TMP2]) return false;
    // ---- commit: where each piece's ids go, the ids, the counts ----
    // (piece totals replaced by their running sum, 256 pieces at a time)
    uint32_t total = 0;
    uint32_t* scan = sm.ws;                     // (the arena is free again)
    for (uint32_t base = 0; base <= K; base += kThreads) {
        blk.par([&](int tid) { const uint32_t k = base + tid; scan[tid] = k <= K ? recs[static_cast<size_t>(k) * kPieceRec] : 0u; });
        uint32_t sum = 0;
        blk.excl_scan(scan, &sum);
        blk.par([&](int tid) { const uint32_t k = base + tid; if (k <= K) recs[static_cast<size_t>(k) * kPieceRec + 1] = total + scan[tid]; });
        total += sum;
    }
    blk.par([&](int tid) {
        // a thread per piece copies its few ids
        for (uint32_t k = tid; k <= K; k += kThreads) {
            const uint32_t* rec = recs + static_cast<size_t>(k) * kPieceRec;
            const uint32_t cnt = rec[0], to = rec[1], from = cuts[k];
            for (uint32_t i = 0; i < cnt; ++i) a.gstage[g + to + i] = piece_ids[from + i];
        }
    });
    blk.par([&](int tid) { if (tid == 0) { a.glong_cnt[li] = total; global_add(a.tile_tok + g / kTile, total); } });
    return true;
}

template <class Blk>
GTOK_DEV void long_word(Blk& blk, const EncodeArgs& a, MissSmem& sm, uint32_t li) {
    const uint32_t n = ldg(a.meta);
    const DeviceTables& tb = a.tb;
    const uint32_t g = ldg(a.glong_g + li);
    uint32_t len = ldg(a.glong_len + li);
    if (len == 0) len = find_word_end(blk, a, sm.ws, g, n) - g;
    blk.par([&](int tid) {
        if (tid != 0) return;
        uint32_t id = kNoToken;
        if (tb.ignore_merges) id = probe_long(tb, a.text, g, len);
        sm.ctr[C_TMP2] = id;
    });
    const uint32_t hit = sm.ctr[C_TMP2];
    if (hit != kNoToken) {
        blk.par([&](int tid) { if (tid == 0) { a.gstage[g] = hit; a.glong_cnt[li] = 1; global_add(a.tile_tok + g / kTile, 1u); } });
        return;
    }
    if (tb.monotone && rle_word(blk, a, sm, li, g, len)) return;
    if (tb.monotone && len >= kPieceMinLen && pieces_word(blk, a, sm, li, g, len)) return;
    // Workspace: shared memory when the pre-token fits beside the team's own scratch,
    // else the per-byte global arrays (disjoint per pre-token).
    constexpr uint32_t kScratch = 6 * kThreads + 16;                 // team scratch + keep buffer
    constexpr uint32_t kFit = (3 * kArenaSyms - kScratch) / 3;
    uint32_t* scratch = sm.ws;
    uint32_t* keepbuf = sm.ws + 3 * kThreads + 16;
    uint32_t *ids, *rk, *nw;
    if (len <= kFit) { ids = sm.ws + kScratch; rk = ids + kFit; nw = rk + kFit; }
    else { ids = a.gstage + g; rk = a.gwork_rk + g; nw = a.gwork_nw + g; }
    blk.par([&](int tid) {
        for (uint32_t i = tid; i < len; i += kThreads) ids[i] = sm.b2i[ldg(a.text + g + i)];
    });
    BlockTeam<Blk> team(blk, keepbuf);
    uint32_t cnt = team_bpe(team, a, ids, rk, nw, len, scratch);
    blk.par([&](int tid) {
        if (ids != a.gstage + g)
            for (uint32_t i = tid; i < cnt; i += kThreads) a.gstage[g + i] = ids[i];
        if (tid == 0) { a.glong_cnt[li] = cnt; global_add(a.tile_tok + g / kTile, cnt); }
    });
}

// ---- kernel 4: output assembly ------------------------------------------------------------
// Each thread keeps its 16 slots in registers from the load to the store: the slots, the
// tile's overflow slots and the earlier tiles' id counts (whose sum is the tile's base) are
// all requested before anything waits, so a tile costs one memory round trip, one block scan
// and the stores.  Beyond kSumTiles tiles the base comes from a look-back chain instead.
template <class Blk>
GTOK_DEV void assemble_tile(Blk& blk, const EncodeArgs& a, AsmSmem& sm, int tile) {
    const uint32_t n = ldg(a.meta);
    const uint32_t n_docs = ldg(a.meta + 1);
    const uint32_t t0 = static_cast<uint32_t>(tile) * kTile;
    const uint32_t n_tiles = (n + kTile - 1) / kTile;
    const uint32_t* ovf = a.ovf + static_cast<size_t>(tile) * kTokExtra;
    const bool direct = n_tiles <= a.sum_tiles;
    struct Slots { uint32_t v[kPer]; };
    typename Blk::template Local<Slots> regs;
    auto mark = [&](int slot) {
        if (!a.phase_clk) return;
        blk.par([&](int tid) {
            if (tid != 0) return;
            unsigned long long t = cycle_now();
            if (slot >= 0) add_cycles(a.phase_clk + slot, t - sm.clk_last);
            sm.clk_last = t;
        });
    };
    mark(-1);
    auto weight = [&](uint32_t v) -> uint32_t {
        if (v == kInvalidTok) return 0u;
        return (v & kLongRef) ? ldg(a.glong_cnt + (v & ~kLongRef)) : 1u;
    };
    // ---- A0: slots into registers; ids per thread; partial sums of the earlier tiles' counts ----
    blk.par([&](int tid) {
        Slots& r = regs.at(tid);
        uint32_t acc = 0;
        if (direct) for (uint32_t j = tid; j < static_cast<uint32_t>(tile); j += kThreads) acc += ldg(a.tile_tok + j);
#if defined(__CUDA_ARCH__)
        const uint4* src = reinterpret_cast<const uint4*>(a.stage + t0) + tid * (kPer / 4);
#pragma unroll
        for (int q = 0; q < kPer / 4; ++q) {
            const uint4 w = ld128(src + q);
            r.v[4 * q] = w.x; r.v[4 * q + 1] = w.y; r.v[4 * q + 2] = w.z; r.v[4 * q + 3] = w.w;
        }
#else
        for (int i = 0; i < kPer; ++i) r.v[i] = a.stage[t0 + tid * kPer + i];
#endif
        uint32_t sum = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < kPer; ++i) sum += weight(r.v[i]);
        sm.scan[tid] = sum;
        sm.sum[tid] = acc;
        if (tid < kTokExtra / 4) {
            uint32_t ex = 0;
            for (int i = 0; i < 4; ++i) { const uint32_t x = ldg(ovf + tid * 4 + i); sm.ovf[tid * 4 + i] = x; ex += x != kInvalidTok; }
            sm.ex[tid] = ex;
        }
        if (tid == 0) sm.ctr[C_NLREF] = 0;
    });
    uint32_t total_main = 0, before = 0;
    blk.excl_scan_and_sum(sm.scan, &total_main, sm.sum, &before);
    uint32_t total = total_main;
    for (int t = 0; t < kTokExtra / 4; ++t) total += sm.ex[t];
    mark(12);
    // ---- A1: tile base ----
    // Every tile's total is known before this kernel starts (tile_tok), so up to kSumTiles tiles a
    // block simply adds up the totals before its own; beyond that (the work is quadratic in the
    // number of tiles) the totals are chained by look-back.
    uint32_t base;
    if (direct) {
        base = before;
        if (ldg(a.tile_tok + tile) != total) blk.par([&](int tid) { if (tid == 0) global_or(a.ctl + CTL_ERR, kErrInternal); });   // the kernels disagree on a count
    } else base = blk.lookback(a.st2, tile, total, a.ctl);
    mark(13);
    // ---- A2: ids to their final place; per-document token offsets ----
    blk.par([&](int tid) {
        const Slots& r = regs.at(tid);
        uint32_t at = base + sm.scan[tid];
        uint32_t docbits = 0;
        if (a.out_doc_tok) {
            const uint32_t p0 = t0 + tid * kPer;
            docbits = (ldg(a.docmask + (p0 >> 5)) >> (p0 & 31)) & 0xFFFFu;
            if (p0 == 0) docbits |= 1u;
        }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < kPer; ++i) {
            const uint32_t v = r.v[i];
            if ((docbits >> i) & 1u) {
                // documents that begin at this byte (several when some are empty): their first id is the next one written
                const uint32_t p = t0 + tid * kPer + i;
                if (p < n) {
                    uint32_t lo = 0, hi = n_docs + 1;
                    while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (ldg(a.doc_off + mid) < p) lo = mid + 1; else hi = mid; }
                    for (uint32_t d = lo; d <= n_docs && ldg(a.doc_off + d) == p; ++d) a.out_doc_tok[d] = at;
                }
            }
            if (v == kInvalidTok) continue;
            if (v & kLongRef) {
                uint32_t li = v & ~kLongRef, slot = shared_add(&sm.ctr[C_NLREF], 1u);
                if (slot < kLongPerTile) { sm.lref_idx[slot] = li; sm.lref_at[slot] = at; }
                at += ldg(a.glong_cnt + li);
                continue;
            }
            if (at < a.out_cap) a.out_tokens[at] = v; else global_or(a.ctl + CTL_ERR, kErrOutputFull);
            ++at;
        }
        if (tid < kTokExtra / 4) {
            at = base + total_main;
            for (int t = 0; t < tid; ++t) at += sm.ex[t];
            for (int i = 0; i < 4; ++i) {
                const uint32_t v = sm.ovf[tid * 4 + i];
                if (v == kInvalidTok) continue;
                if (at < a.out_cap) a.out_tokens[at] = v; else global_or(a.ctl + CTL_ERR, kErrOutputFull);
                ++at;
            }
        }
    });
    {
        uint32_t n_ref = sm.ctr[C_NLREF];
        if (n_ref > kLongPerTile) n_ref = kLongPerTile;
        if (n_ref) {
            blk.par([&](int tid) {
                for (uint32_t r = 0; r < n_ref; ++r) {
                    const uint32_t li = sm.lref_idx[r], at = sm.lref_at[r];
                    const uint32_t g = ldg(a.glong_g + li), cnt = ldg(a.glong_cnt + li);
                    for (uint32_t i = tid; i < cnt; i += kThreads) {
                        if (at + i < a.out_cap) a.out_tokens[at + i] = a.gstage[g + i];
                        else { global_or(a.ctl + CTL_ERR, kErrOutputFull); break; }
                    }
                }
            });
        }
    }
    mark(14);
    // ---- A3: offsets of the documents past the text's end; total ----
    if (static_cast<uint32_t>(tile) + 1 == n_tiles) {
        blk.par([&](int tid) {
            if (a.out_doc_tok) {
                uint32_t lo2 = 0, hi2 = n_docs + 1;
                while (lo2 < hi2) { uint32_t mid = (lo2 + hi2) >> 1; if (ldg(a.doc_off + mid) < n) lo2 = mid + 1; else hi2 = mid; }
                for (uint32_t d = lo2 + tid; d <= n_docs; d += kThreads) a.out_doc_tok[d] = base + total;
            }
            if (tid == 0) a.status[0] = base + total;
        });
    }
    mark(15);
}

}  // namespace gtok
