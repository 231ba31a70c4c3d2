"""ctypes bindings for the test-side checkers: the CPU oracle (oracle/liboracle.so),
the reference's own host encoder when it was built (oracle/_ref/libgtok_ref.so) and
the serial emulation of the kernels (tests/cpu_emul/libemul.so).  Test infrastructure
only; nothing in the shipped package imports this module."""
import ctypes
import os
import subprocess
import unicodedata

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libgtok_ref.so")
EMUL_DIR = os.path.join(ROOT, "tests", "cpu_emul")
EMUL_SO = os.path.join(EMUL_DIR, "libemul.so")
CSRC = os.path.join(ROOT, "graphtok_b200", "csrc")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_oracle():
    deps = [os.path.join(ORACLE_DIR, "gtok_oracle.cc")] + [os.path.join(CSRC, f) for f in ("vocab_host.cc", "vocab_host.h", "json_min.h", "unicode_class_table.h")]
    if _stale(ORACLE_SO, deps):
        subprocess.run(["make", "-C", ORACLE_DIR, "oracle"], check=True, stdout=subprocess.DEVNULL)
    return ORACLE_SO


def reference_dir():
    """Checkout of the reference project: $GTOK_REFERENCE_DIR, else a directory `reference` beside this
    repository; None when neither holds its sources."""
    for d in (os.environ.get("GTOK_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if d and os.path.isdir(os.path.join(d, "src")):
            return d
    return None


def build_ref():
    """Builds the reference host encoder when its sources are present; returns the path or None."""
    ref = reference_dir()
    if ref and _stale(REF_SO, [os.path.join(ORACLE_DIR, "ref_wrapper.cc")]):
        subprocess.run(["make", "-C", ORACLE_DIR, "ref", "REF=" + ref], check=True, stdout=subprocess.DEVNULL)
    return REF_SO if os.path.exists(REF_SO) else None


def build_emul():
    deps = [os.path.join(EMUL_DIR, "emul.cc")] + [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    if _stale(EMUL_SO, deps):
        subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-o", EMUL_SO, os.path.join(EMUL_DIR, "emul.cc"),
                        os.path.join(CSRC, "vocab_host.cc"), os.path.join(CSRC, "tables_build.cc"), os.path.join(CSRC, "nfc_host.cc")], check=True)
    return EMUL_SO


def nfc(data):
    """NFC of UTF-8 bytes (Python unicodedata, Unicode 15.0, which Hugging Face tokenizers agrees with)."""
    return unicodedata.normalize("NFC", data.decode("utf-8")).encode("utf-8")


def lib_nfc(data):
    """NFC by the library's own host code (csrc/nfc_host.cc), for checking it against `nfc`."""
    lib = ctypes.CDLL(build_emul())
    lib.gtok_emul_nfc.restype = ctypes.c_int64
    lib.gtok_emul_nfc.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint64]
    out = ctypes.create_string_buffer(len(data) * 3 + 16)
    n = lib.gtok_emul_nfc(bytes(data), len(data), out, len(out))
    assert n >= 0
    return out.raw[:n]


def device_nfc(data, doc_off=None, reverse=False, cap=None, already_normalised=False):
    """NFC by the device normaliser's tile program (csrc/nfc_core.h) run on the CPU.  Returns the bytes, or
    (bytes, new offsets) when `doc_off` is given; a negative kernel status is returned as an int."""
    lib = ctypes.CDLL(build_emul())
    f = lib.gtok_emul_nfc_device
    f.restype = ctypes.c_int64
    f.argtypes = [ctypes.c_char_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_char_p, ctypes.c_uint32,
                  ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    data = bytes(data)
    cap = len(data) * 3 + 64 if cap is None else cap
    out = ctypes.create_string_buffer(cap + 64)
    if doc_off is None:
        n = f(data, len(data), None, 1, out, cap, None, int(reverse), int(already_normalised))
        return out.raw[:n] if n >= 0 else int(n)
    offs = (ctypes.c_uint32 * len(doc_off))(*doc_off)
    new = (ctypes.c_uint32 * len(doc_off))()
    n = f(data, len(data), offs, len(doc_off) - 1, out, cap, new, int(reverse), int(already_normalised))
    return (out.raw[:n], list(new)) if n >= 0 else int(n)


class Oracle:
    def __init__(self, tokenizer_json):
        self.lib = ctypes.CDLL(build_oracle())
        self.lib.gtok_oracle_create.restype = ctypes.c_void_p
        self.lib.gtok_oracle_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
        self.lib.gtok_oracle_encode.restype = ctypes.c_int64
        self.lib.gtok_oracle_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64,
                                                ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        self.lib.gtok_oracle_family.restype = ctypes.c_uint32
        self.lib.gtok_oracle_family.argtypes = [ctypes.c_void_p]
        self.lib.gtok_oracle_destroy.argtypes = [ctypes.c_void_p]
        err = ctypes.create_string_buffer(512)
        self.h = self.lib.gtok_oracle_create(os.fsencode(tokenizer_json), err, 512)
        if not self.h:
            raise RuntimeError("oracle: " + err.value.decode())
        self.needs_nfc = bool(self.lib.gtok_oracle_family(self.h) & 0x100)

    def encode_normalized(self, data, want_starts=False):
        data = bytes(data)
        out = np.empty(len(data) + 8, dtype=np.uint32)
        if want_starts:
            st = np.empty(len(data) + 8, dtype=np.uint32)
            ns = ctypes.c_uint64(0)
            n = self.lib.gtok_oracle_encode(self.h, data, len(data), out.ctypes.data, out.size, st.ctypes.data, st.size, ctypes.byref(ns))
            return out[:n].copy(), st[:ns.value].copy()
        n = self.lib.gtok_oracle_encode(self.h, data, len(data), out.ctypes.data, out.size, None, 0, None)
        return out[:n].copy()

    def encode(self, data):
        """Full path as the reference's CPU route does it: normalise (Qwen2.5), then encode."""
        return self.encode_normalized(nfc(data) if self.needs_nfc else data)

    def encode_batch(self, blob, offsets):
        ids, offs = [], [0]
        for i in range(len(offsets) - 1):
            t = self.encode(blob[int(offsets[i]):int(offsets[i + 1])])
            ids.append(t)
            offs.append(offs[-1] + len(t))
        return (np.concatenate(ids) if ids else np.zeros(0, np.uint32)), np.array(offs, dtype=np.uint32)


class Reference:
    """The reference's HostEncoder, compiled from its own sources (oracle/_ref)."""

    def __init__(self, tokenizer_json):
        so = build_ref()
        if not so:
            raise FileNotFoundError(REF_SO)
        self.lib = ctypes.CDLL(so)
        self.lib.gtok_ref_create.restype = ctypes.c_void_p
        self.lib.gtok_ref_create.argtypes = [ctypes.c_char_p]
        self.lib.gtok_ref_encode.restype = ctypes.c_int64
        self.lib.gtok_ref_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64]
        self.h = self.lib.gtok_ref_create(os.fsencode(tokenizer_json))
        if not self.h:
            raise RuntimeError("reference loader rejected " + tokenizer_json)

    def encode_normalized(self, data):
        data = bytes(data)
        out = np.empty(len(data) + 8, dtype=np.uint32)
        n = self.lib.gtok_ref_encode(self.h, data, len(data), out.ctypes.data, out.size)
        return out[:n].copy()


class Emul:
    """Kernels' tile programs run serially on the CPU (tests/cpu_emul/emul.cc)."""

    def __init__(self, tokenizer_json):
        self.lib = ctypes.CDLL(build_emul())
        self.lib.gtok_emul_create.restype = ctypes.c_void_p
        self.lib.gtok_emul_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
        self.lib.gtok_emul_encode.restype = ctypes.c_int64
        self.lib.gtok_emul_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                              ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        err = ctypes.create_string_buffer(512)
        self.h = self.lib.gtok_emul_create(os.fsencode(tokenizer_json), err, 512)
        if not self.h:
            raise RuntimeError("emul: " + err.value.decode())

    def encode(self, data, offsets=None, reverse=False, non_monotone=False, want_starts=False, trie=False):
        data = bytes(data)
        out = np.empty(len(data) + 16, dtype=np.uint32)
        bm = np.zeros((len(data) + 4095) // 4096 * 128 + 8, dtype=np.uint32)
        doc = None
        if offsets is not None:
            offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
            doc = np.zeros(offsets.size, dtype=np.uint32)
            n = self.lib.gtok_emul_encode(self.h, data, len(data), offsets.ctypes.data, offsets.size - 1, out.ctypes.data, out.size,
                                          doc.ctypes.data, bm.ctypes.data, int(reverse), int(non_monotone) | (2 if trie else 0))
        else:
            n = self.lib.gtok_emul_encode(self.h, data, len(data), None, 1, out.ctypes.data, out.size, None, bm.ctypes.data,
                                          int(reverse), int(non_monotone) | (2 if trie else 0))
        if n < 0:
            raise RuntimeError("emulated kernels flagged error bits %d" % -n)
        ids = out[:n].copy()
        res = [ids]
        if offsets is not None:
            res.append(doc)
        if want_starts:
            bits = np.unpackbits(bm.view(np.uint8), bitorder="little")[:len(data)]
            res.append(np.nonzero(bits)[0].astype(np.uint32))
        return res[0] if len(res) == 1 else tuple(res)

    def decode(self, ids, cap=None, reverse=False):
        """decode_tile over the ids; returns (bytes or None when `cap` is too small, byte count, error bits)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        f = self.lib.gtok_emul_decode
        f.restype = ctypes.c_int64
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p]
        if cap is None:
            cap = 64 * ids.size + 64
        out = np.zeros(cap + 16, dtype=np.uint8)
        bits = ctypes.c_uint32(0)
        total = f(self.h, ids.ctypes.data, ids.size, out.ctypes.data, cap, int(reverse), ctypes.byref(bits))
        ok = total <= cap and not (bits.value & 1)
        return (out[:total].tobytes() if ok else None), int(total), bits.value


def token_spellings(tokenizer_json):
    """id -> raw bytes, straight from the tokenizer.json: model vocabulary strings mapped back
    through the GPT-2 byte-to-unicode table (the reference's gpt2_token_decoded_bytes,
    src/vocab.h:25-28), added tokens as their UTF-8 content.  Decoding oracle."""
    import json
    cs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    back = {}
    extra = 0
    for b in range(256):
        if b in cs:
            back[chr(b)] = b
        else:
            back[chr(256 + extra)] = b
            extra += 1
    j = json.load(open(tokenizer_json, encoding="utf-8"))
    table = {}
    if j["model"].get("byte_fallback"):
        # the Gemma-3 shape: raw strings, U+2581 for a space, "<0xNN>" for a byte (its decoder section says the same)
        import re
        for tok, tid in j["model"]["vocab"].items():
            m = re.fullmatch(r"<0x([0-9A-F]{2})>", tok)
            table[tid] = bytes([int(m.group(1), 16)]) if m else tok.replace("\u2581", " ").encode("utf-8")
        for at in j.get("added_tokens", []):
            table[at["id"]] = at["content"].encode("utf-8")
        return table
    for tok, tid in j["model"]["vocab"].items():
        table[tid] = bytes(back[ch] for ch in tok)
    for at in j.get("added_tokens", []):
        table[at["id"]] = at["content"].encode("utf-8")
    return table
