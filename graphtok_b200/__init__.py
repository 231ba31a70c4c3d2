"""B200-native encode path behind the libgtok C ABI.

The product is `lib/libgtok.so` (CUDA kernels + C++ engine + extern "C" boundary,
built by `python -m graphtok_b200.build`).  This package only locates and binds it
through ctypes; it has no CPU implementation of the encode path, and `GTok(...)`
raises when the library or a B200 is missing.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libgtok.so")

_lib = None


def plan_documents(offsets, n_parts):
    """Contiguous document ranges of about equal bytes: n_parts + 1 document indices."""
    offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
    out = np.zeros(n_parts + 1, dtype=np.uint32)
    if load_lib().gtok_x_plan_documents(offsets.ctypes.data, offsets.size - 1, n_parts, out.ctypes.data) != 0:
        raise RuntimeError("gtok_x_plan_documents failed")
    return out


def load_lib():
    """ctypes handle on libgtok.so with argument/return types declared."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libgtok.so is not built: run `python -m graphtok_b200.build` (%s)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    vp, u32, i32, cp = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int32, ctypes.c_char_p
    lib.gtok_create.restype = vp
    lib.gtok_create.argtypes = [cp, u32]
    lib.gtok_encode.restype = i32
    lib.gtok_encode.argtypes = [vp, vp, u32, vp, u32]
    lib.gtok_encode_to_device.restype = i32
    lib.gtok_encode_to_device.argtypes = [vp, vp, u32, vp, u32]
    lib.gtok_encode_batch.restype = i32
    lib.gtok_encode_batch.argtypes = [vp, vp, vp, u32, vp, u32, vp]
    lib.gtok_cpu_max_bytes.restype = u32
    lib.gtok_cpu_max_bytes.argtypes = [vp]
    lib.gtok_set_cpu_max_bytes.restype = None
    lib.gtok_set_cpu_max_bytes.argtypes = [vp, u32]
    lib.gtok_cpu_backend.restype = cp
    lib.gtok_cpu_backend.argtypes = [vp]
    lib.gtok_dispatcher_create.restype = vp
    lib.gtok_dispatcher_create.argtypes = [cp, u32, u32, u32, u32]
    lib.gtok_dispatch_encode.restype = i32
    lib.gtok_dispatch_encode.argtypes = [vp, vp, u32, vp, u32]
    lib.gtok_dispatcher_stats.restype = None
    lib.gtok_dispatcher_stats.argtypes = [vp, vp]
    lib.gtok_dispatcher_destroy.restype = None
    lib.gtok_dispatcher_destroy.argtypes = [vp]
    lib.gtok_vocab_size.restype = u32
    lib.gtok_vocab_size.argtypes = [vp]
    lib.gtok_destroy.restype = None
    lib.gtok_destroy.argtypes = [vp]
    lib.gtok_x_last_error.restype = cp
    lib.gtok_x_last_error.argtypes = []
    lib.gtok_x_family.restype = u32
    lib.gtok_x_family.argtypes = [vp]
    lib.gtok_x_stage.restype = i32
    lib.gtok_x_stage.argtypes = [vp, vp, u32, vp, u32]
    lib.gtok_x_replay.restype = i32
    lib.gtok_x_replay.argtypes = [vp, vp]
    lib.gtok_x_read.restype = i32
    lib.gtok_x_read.argtypes = [vp, vp, u32, vp]
    lib.gtok_x_read_boundaries.restype = i32
    lib.gtok_x_read_boundaries.argtypes = [vp, vp, u32]
    lib.gtok_x_boundaries_noalloc.restype = i32
    lib.gtok_x_boundaries_noalloc.argtypes = [vp, vp, u32, vp, vp]
    lib.gtok_x_phase_clocks.restype = i32
    lib.gtok_x_phase_clocks.argtypes = [vp, vp, i32]
    lib.gtok_x_encode_batch_to_device.restype = i32
    lib.gtok_x_encode_batch_to_device.argtypes = [vp, vp, vp, u32, vp, u32, vp]
    lib.gtok_x_set_max_bytes.restype = u32
    lib.gtok_x_set_max_bytes.argtypes = [vp, u32]
    lib.gtok_x_work_stats.restype = i32
    lib.gtok_x_work_stats.argtypes = [vp, vp]
    lib.gtok_x_timeline.restype = i32
    lib.gtok_x_timeline.argtypes = [vp, vp, u32]
    lib.gtok_x_token_bytes.restype = i32
    lib.gtok_x_token_bytes.argtypes = [vp, u32, vp, u32]
    lib.gtok_x_decode.restype = ctypes.c_int64
    lib.gtok_x_decode.argtypes = [vp, vp, u32, vp, ctypes.c_uint64, vp, vp]
    lib.gtok_x_profile.restype = i32
    lib.gtok_x_profile.argtypes = [vp, vp]
    lib.gtok_x_plan_chunks.restype = i32
    lib.gtok_x_plan_chunks.argtypes = [vp, vp, ctypes.c_uint64, u32, vp]
    lib.gtok_x_plan_documents.restype = i32
    lib.gtok_x_plan_documents.argtypes = [vp, u32, u32, vp]
    lib.gtok_x_table_bytes.restype = None
    lib.gtok_x_table_bytes.argtypes = [vp, vp]
    lib.gtok_x_launches_per_replay.restype = i32
    lib.gtok_x_launches_per_replay.argtypes = [vp, i32]
    _lib = lib
    return lib


class GTokError(RuntimeError):
    pass


class GTok:
    """Thin object over one libgtok handle (not thread-safe, like the handle)."""

    def __init__(self, tokenizer_json, max_bytes=1 << 20):
        self.lib = load_lib()
        self.handle = self.lib.gtok_create(os.fsencode(tokenizer_json), int(max_bytes))
        if not self.handle:
            raise GTokError("gtok_create failed: %s" % self.lib.gtok_x_last_error().decode("utf-8", "replace"))
        self.max_bytes = max(4096, int(max_bytes))

    def set_max_bytes(self, max_bytes):
        """Raises the handle's byte cap in place (tables stay; the context grows when next needed)."""
        self.max_bytes = int(self.lib.gtok_x_set_max_bytes(self.handle, int(max_bytes)))
        return self.max_bytes

    def close(self):
        if getattr(self, "handle", None):
            self.lib.gtok_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _fail(self, what, code):
        raise GTokError("%s returned %d: %s" % (what, code, self.lib.gtok_x_last_error().decode("utf-8", "replace")))

    def encode(self, data):
        """bytes -> uint32 ids (numpy)."""
        data = bytes(data)
        out = np.empty(len(data) + 16, dtype=np.uint32)
        n = self.lib.gtok_encode(self.handle, data, len(data), out.ctypes.data, out.size)
        if n == -2:
            # more ids than bytes: only text that its vocabulary's NFC lengthens (at most threefold)
            out = np.empty(3 * len(data) + 64, dtype=np.uint32)
            n = self.lib.gtok_encode(self.handle, data, len(data), out.ctypes.data, out.size)
        if n < 0:
            self._fail("gtok_encode", n)
        return out[:n].copy()

    def encode_batch(self, blob, offsets):
        """Concatenated documents + n+1 byte offsets -> (ids uint32[T], token offsets uint32[n+1])."""
        blob = bytes(blob)
        offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
        n_docs = offsets.size - 1
        out = np.empty(len(blob) + 16, dtype=np.uint32)
        doc = np.empty(n_docs + 1, dtype=np.uint32)
        n = self.lib.gtok_encode_batch(self.handle, blob, offsets.ctypes.data, n_docs, out.ctypes.data, out.size, doc.ctypes.data)
        if n == -2:
            # more ids than bytes: only text that its vocabulary's NFC lengthens (at most threefold)
            out = np.empty(3 * len(blob) + 64, dtype=np.uint32)
            n = self.lib.gtok_encode_batch(self.handle, blob, offsets.ctypes.data, n_docs, out.ctypes.data, out.size, doc.ctypes.data)
        if n < 0:
            self._fail("gtok_encode_batch", n)
        return out[:n].copy(), doc

    # ---- measurement -----------------------------------------------------
    def stage(self, blob, offsets=None):
        blob = bytes(blob)
        if offsets is None:
            r = self.lib.gtok_x_stage(self.handle, blob, len(blob), None, 1)
        else:
            offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
            r = self.lib.gtok_x_stage(self.handle, blob, len(blob), offsets.ctypes.data, offsets.size - 1)
        if r < 0:
            self._fail("gtok_x_stage", r)

    def replay(self):
        """One graph replay of the staged input: (token count, milliseconds on the device)."""
        ms = ctypes.c_float(0.0)
        n = self.lib.gtok_x_replay(self.handle, ctypes.byref(ms))
        if n < 0:
            self._fail("gtok_x_replay", n)
        return n, ms.value

    def read(self, n_tokens, n_docs=None):
        out = np.empty(n_tokens + 16, dtype=np.uint32)
        doc = np.empty((n_docs or 0) + 1, dtype=np.uint32)
        n = self.lib.gtok_x_read(self.handle, out.ctypes.data, out.size, doc.ctypes.data if n_docs else None)
        if n < 0:
            self._fail("gtok_x_read", n)
        return out[:n].copy(), (doc if n_docs else None)

    def boundaries(self, n_bytes):
        """Byte offsets at which pre-tokens start, for the staged input after a replay."""
        words = np.zeros((n_bytes + 31) // 32 + 1, dtype=np.uint32)
        r = self.lib.gtok_x_read_boundaries(self.handle, words.ctypes.data, words.size)
        if r < 0:
            self._fail("gtok_x_read_boundaries", r)
        bits = np.unpackbits(words.view(np.uint8), bitorder="little")[:n_bytes]
        return np.nonzero(bits)[0].astype(np.uint32)

    def profile(self):
        """Staged input, kernel by kernel: (tokens, pretok ms, words ms, miss ms, assemble ms, sequence ms,
        ms of what runs before pretok: normalisation and document-bit kernels)."""
        ms = (ctypes.c_float * 6)()
        n = self.lib.gtok_x_profile(self.handle, ms)
        if n < 0:
            self._fail("gtok_x_profile", n)
        return (n,) + tuple(ms)

    def decode(self, ids, out=None, want_ms=False):
        """ids -> the bytes they spell, on the device (gtok_x_decode).  `out`: optional uint8 numpy
        buffer to decode into (a page-locked one is written directly); returns bytes, or with
        `want_ms` (bytes, CUDA-event ms of the decode graph)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        need = ctypes.c_uint64(0)
        ms = ctypes.c_float(0.0)
        buf = out if out is not None else np.empty(16 * ids.size + 1024, dtype=np.uint8)
        n = self.lib.gtok_x_decode(self.handle, ids.ctypes.data, ids.size, buf.ctypes.data, buf.size, ctypes.byref(need), ctypes.byref(ms))
        if n == -2 and out is None:
            buf = np.empty(need.value, dtype=np.uint8)
            n = self.lib.gtok_x_decode(self.handle, ids.ctypes.data, ids.size, buf.ctypes.data, buf.size, ctypes.byref(need), ctypes.byref(ms))
        if n < 0:
            self._fail("gtok_x_decode", n)
        data = buf[:n].tobytes()
        return (data, ms.value) if want_ms else data

    def plan_chunks(self, data, n_parts):
        data = bytes(data)
        out = np.zeros(n_parts + 1, dtype=np.uint64)
        if self.lib.gtok_x_plan_chunks(self.handle, data, len(data), n_parts, out.ctypes.data) != 0:
            raise GTokError("gtok_x_plan_chunks failed")
        return out

    def work_stats(self):
        """After a replay of the staged input: dict of what went from kernel to kernel (gtok_x_work_stats)."""
        v = (ctypes.c_uint64 * 6)()
        if self.lib.gtok_x_work_stats(self.handle, v) != 0:
            raise GTokError("gtok_x_work_stats failed")
        keys = ("pretokens", "unknown_pretokens", "unknown_bytes", "long_pretokens", "long_bytes", "ids_from_miss_kernel")
        return dict(zip(keys, (int(x) for x in v)))

    def table_bytes(self):
        t = (ctypes.c_uint64 * 3)()
        self.lib.gtok_x_table_bytes(self.handle, t)
        return int(t[0]), int(t[1]), int(t[2])

    def family(self):
        return self.lib.gtok_x_family(self.handle)
