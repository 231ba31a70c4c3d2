// TEST INFRASTRUCTURE ONLY.  C entry points around the reference's own host
// encoder (src/host_encode.cc HostEncoder, src/vocab.cc load_hf_tokenizer_json),
// compiled from the reference's sources where they lie by oracle/Makefile into
// oracle/_ref/libgtok_ref.so.  No reference source is copied into this tree.
// Used to pin the restatement in gtok_oracle.cc and, optionally, as the timed
// CPU baseline.  The encoder takes bytes that are already normalised
// (src/host_encode.h:44-45); the caller applies NFC first for Qwen2.5.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "host_encode.h"
#include "vocab.h"
#include <utf8proc.h>

namespace {
struct RefHandle {
    gbpe::HostVocab hv;
    gbpe::HostEncoder* enc = nullptr;
    std::vector<uint32_t> out;
};
[[noreturn]] void unreachable_shim(const char* what) {
    std::fprintf(stderr, "ref_wrapper: utf8proc stand-in %s called; the wrapper never normalises\n", what);
    std::abort();
}
}  // namespace

extern "C" {

// utf8proc stand-ins: never called (see shim/utf8proc.h).
const utf8proc_property_t* utf8proc_get_property(utf8proc_int32_t) { unreachable_shim("get_property"); }
utf8proc_ssize_t utf8proc_decompose_char(utf8proc_int32_t, utf8proc_int32_t*, utf8proc_ssize_t, utf8proc_option_t, int*) { unreachable_shim("decompose_char"); }
utf8proc_ssize_t utf8proc_normalize_utf32(utf8proc_int32_t*, utf8proc_ssize_t, utf8proc_option_t) { unreachable_shim("normalize_utf32"); }
utf8proc_ssize_t utf8proc_iterate(const utf8proc_uint8_t*, utf8proc_ssize_t, utf8proc_int32_t*) { unreachable_shim("iterate"); }
utf8proc_ssize_t utf8proc_decompose(const utf8proc_uint8_t*, utf8proc_ssize_t, utf8proc_int32_t*, utf8proc_ssize_t, utf8proc_option_t) { unreachable_shim("decompose"); }
utf8proc_ssize_t utf8proc_reencode(utf8proc_int32_t*, utf8proc_ssize_t, utf8proc_option_t) { unreachable_shim("reencode"); }
const char* utf8proc_errmsg(utf8proc_ssize_t) { return "utf8proc stand-in"; }

void* gtok_ref_create(const char* tokenizer_json) {
    RefHandle* h = new RefHandle();
    if (!gbpe::load_hf_tokenizer_json(tokenizer_json, h->hv)) { delete h; return nullptr; }
    h->enc = new gbpe::HostEncoder(h->hv);
    if (!h->enc->supported()) { delete h->enc; delete h; return nullptr; }
    return h;
}

void gtok_ref_destroy(void* p) {
    RefHandle* h = static_cast<RefHandle*>(p);
    if (!h) return;
    delete h->enc;
    delete h;
}

// Returns the token count; writes at most `cap` ids.
int64_t gtok_ref_encode(void* p, const uint8_t* text, uint64_t len, uint32_t* out, uint64_t cap) {
    RefHandle* h = static_cast<RefHandle*>(p);
    h->enc->encode(text, static_cast<size_t>(len), h->out);
    uint64_t w = h->out.size() < cap ? h->out.size() : cap;
    if (out && w) std::memcpy(out, h->out.data(), w * sizeof(uint32_t));
    return static_cast<int64_t>(h->out.size());
}

}  // extern "C"
