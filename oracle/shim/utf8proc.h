// TEST INFRASTRUCTURE ONLY.  Stand-in for <utf8proc.h>, which is not installed
// here.  It declares the handful of names the reference's src/vocab.cc uses so
// that file compiles with its Qwen2.5 loader enabled; the functions are
// defined in ref_wrapper.cc and abort when called.  The wrapper only ever
// hands the reference encoder bytes that are already NFC-normalised, so the
// reference's normaliser (and with it every function below) is never reached.
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef int32_t utf8proc_int32_t;
typedef uint8_t utf8proc_uint8_t;
typedef int16_t utf8proc_int16_t;
typedef uint16_t utf8proc_uint16_t;
typedef ptrdiff_t utf8proc_ssize_t;
typedef int16_t utf8proc_propval_t;
typedef enum {
  UTF8PROC_NULLTERM = (1 << 0), UTF8PROC_STABLE = (1 << 1), UTF8PROC_COMPAT = (1 << 2),
  UTF8PROC_COMPOSE = (1 << 3), UTF8PROC_DECOMPOSE = (1 << 4)
} utf8proc_option_t;
typedef struct utf8proc_property_struct {
  utf8proc_propval_t category;
  utf8proc_propval_t combining_class;
  utf8proc_propval_t bidi_class;
  utf8proc_propval_t decomp_type;
  utf8proc_uint16_t decomp_seqindex;
  utf8proc_uint16_t casefold_seqindex;
  utf8proc_uint16_t uppercase_seqindex;
  utf8proc_uint16_t lowercase_seqindex;
  utf8proc_uint16_t titlecase_seqindex;
  utf8proc_uint16_t comb_index;
} utf8proc_property_t;
const utf8proc_property_t* utf8proc_get_property(utf8proc_int32_t cp);
utf8proc_ssize_t utf8proc_decompose_char(utf8proc_int32_t cp, utf8proc_int32_t* dst, utf8proc_ssize_t bufsize,
                                         utf8proc_option_t options, int* last_boundclass);
utf8proc_ssize_t utf8proc_normalize_utf32(utf8proc_int32_t* buffer, utf8proc_ssize_t length, utf8proc_option_t options);
utf8proc_ssize_t utf8proc_iterate(const utf8proc_uint8_t* str, utf8proc_ssize_t strlen, utf8proc_int32_t* codepoint_ref);
utf8proc_ssize_t utf8proc_decompose(const utf8proc_uint8_t* str, utf8proc_ssize_t strlen, utf8proc_int32_t* buffer,
                                    utf8proc_ssize_t bufsize, utf8proc_option_t options);
utf8proc_ssize_t utf8proc_reencode(utf8proc_int32_t* buffer, utf8proc_ssize_t length, utf8proc_option_t options);
const char* utf8proc_errmsg(utf8proc_ssize_t errcode);
#ifdef __cplusplus
}
#endif
