"""`gpu_bpe_tokenizer` — the reference's Python surface (src/python_bindings.cc:1188-1386,
python/gpu_bpe_tokenizer/__init__.py) over this repository's libgtok.so.

Same class and method names, argument meaning and return types: `Tokenizer.encode`,
`encode_numpy`, `encode_batch` (uint32 tokens and uint32 offsets; `[]` gives `([], [0])`),
`encode_to_device`, `decode`, the `bench_*` helpers and the read-only properties;
`Dispatcher.encode_numpy` / `stats()`.  Every encode runs on the GPU: there is no CPU route,
so `cpu_backend` is "off", `host_max_bytes` reads 0 and `last_route` is always "gpu".

The repository root also carries a package `gpu_bpe_tokenizer` that re-exports this module, so that
a caller's `import gpu_bpe_tokenizer` works unchanged with the repository root on sys.path.
"""
import ctypes
import os

import numpy as np

from .. import GTok, GTokError, load_lib

__all__ = ["Tokenizer", "Dispatcher"]

_KINDS = {0: "GPT2", 1: "Llama3", 2: "Qwen25", 3: "DeepSeekV3", 4: "Gemma3"}
_POLICIES = {"adaptive": 0, "gpu": 1, "cpu": 2}
_BACKENDS = ("", "auto", "off", "host", "gigatoken")


def _as_bytes(text):
    if isinstance(text, str):
        return text.encode("utf-8")
    if isinstance(text, (bytes, bytearray, memoryview)):
        return bytes(text)
    raise TypeError("text must be str or bytes")


class Tokenizer:
    """One vocabulary, one GPU.  Not thread-safe (same contract as the reference, :1117-1120)."""

    def __init__(self, vocab_path, max_input_chars=4096, enable_decode=True, host_max_bytes=None, cpu_backend=""):
        if cpu_backend not in _BACKENDS:
            raise ValueError("cpu_backend must be one of '', 'auto', 'off', 'host', 'gigatoken'")
        self._path = os.fspath(vocab_path)
        self._cap = max(4096, int(max_input_chars))
        self._g = GTok(self._path, max_bytes=self._cap)
        self._decode = bool(enable_decode)
        self._staged_docs = None

    # ---- capacity ------------------------------------------------------------
    def _ensure(self, n_bytes):
        """The C ABI answers -3 above the handle's byte cap and leaves growing to the caller: the cap
        is raised in place (gtok_x_set_max_bytes), the vocabulary and its tables stay as they are."""
        if n_bytes > self._cap:
            cap = self._cap
            while cap < n_bytes:
                cap *= 2
            self._cap = self._g.set_max_bytes(cap)

    # ---- encode --------------------------------------------------------------
    def encode_numpy(self, text):
        data = _as_bytes(text)
        self._ensure(len(data) * 3 + 64)        # NFC lengthens a text at most threefold
        return self._g.encode(data)

    def encode(self, text):
        return self.encode_numpy(text).tolist()

    __call__ = encode

    def encode_batch(self, texts):
        texts = list(texts)
        if not texts:
            return np.zeros(0, dtype=np.uint32), np.zeros(1, dtype=np.uint32)
        blobs = [_as_bytes(t) for t in texts]
        offs = np.zeros(len(blobs) + 1, dtype=np.uint32)
        np.cumsum([len(b) for b in blobs], out=offs[1:])
        self._ensure(int(offs[-1]) * 3 + 64)
        return self._g.encode_batch(b"".join(blobs), offs)

    def encode_to_device(self, text):
        """int32 torch tensor on the GPU (torch is imported only here, as in the reference :100-117)."""
        import torch
        data = _as_bytes(text)
        self._ensure(len(data) * 3 + 64)
        out = torch.empty(len(data) + 16, dtype=torch.int32, device="cuda")
        n = self._g.lib.gtok_encode_to_device(self._g.handle, data, len(data), ctypes.c_void_p(out.data_ptr()), out.numel())
        if n == -2:                                 # text its vocabulary's NFC lengthens
            out = torch.empty(3 * len(data) + 64, dtype=torch.int32, device="cuda")
            n = self._g.lib.gtok_encode_to_device(self._g.handle, data, len(data), ctypes.c_void_p(out.data_ptr()), out.numel())
        if n < 0:
            raise RuntimeError("gtok_encode_to_device returned %d" % n)
        return out[:n]

    def encode_batch_to_device(self, texts):
        """(int32 ids, int32 n+1 token offsets) as torch tensors on the GPU, copied device to device."""
        import torch
        blobs = [_as_bytes(t) for t in texts]
        if not blobs:
            return torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
        offs = np.zeros(len(blobs) + 1, dtype=np.uint32)
        np.cumsum([len(b) for b in blobs], out=offs[1:])
        total = int(offs[-1])
        self._ensure(total * 3 + 64)
        blob = b"".join(blobs)
        doc = torch.empty(len(blobs) + 1, dtype=torch.int32, device="cuda")
        for room in (total + 16, 3 * total + 64):
            out = torch.empty(room, dtype=torch.int32, device="cuda")
            n = self._g.lib.gtok_x_encode_batch_to_device(self._g.handle, blob, offs.ctypes.data, len(blobs), ctypes.c_void_p(out.data_ptr()), out.numel(),
                                                          ctypes.c_void_p(doc.data_ptr()))
            if n != -2:
                break
        if n < 0:
            raise RuntimeError("gtok_x_encode_batch_to_device returned %d" % n)
        return out[:n], doc

    # ---- decode (on the device: ids -> the tokens' bytes, gtok_x_decode) ---------
    def decode_bytes(self, ids):
        if not self._decode:
            raise RuntimeError("decode() is disabled; construct Tokenizer(..., enable_decode=True)")
        arr = np.asarray(ids)
        if arr.size and (arr.min() < 0 or arr.max() > 0xFFFFFFFF):
            raise ValueError("token ids must fit 32 unsigned bits")
        return self._g.decode(arr.astype(np.uint32, copy=False))

    def decode(self, ids):
        return self.decode_bytes(ids).decode("utf-8")          # strict, as the reference (PyUnicode_DecodeUTF8 "strict")

    # ---- measurement helpers (graph replays on staged input) --------------------
    def bench_stage(self, text):
        data = _as_bytes(text)
        self._ensure(len(data) + 16)
        self._g.stage(data)
        self._staged_docs = None

    def bench_run(self):
        """One replay: (token count, device milliseconds)."""
        return self._g.replay()

    def bench_stage_batch(self, texts):
        blobs = [_as_bytes(t) for t in texts]
        offs = np.zeros(len(blobs) + 1, dtype=np.uint32)
        np.cumsum([len(b) for b in blobs], out=offs[1:])
        self._ensure(int(offs[-1]) + 16)
        self._g.stage(b"".join(blobs), offs)
        self._staged_docs = len(blobs)

    bench_run_batch = bench_run

    def bench_readback_batch(self):
        n, _ = self._g.replay()
        return self._g.read(n, self._staged_docs)

    # ---- properties ----------------------------------------------------------------
    @property
    def host_max_bytes(self):
        return 0

    @host_max_bytes.setter
    def host_max_bytes(self, value):      # accepted and ignored: there is no CPU route
        pass

    host_max_bytes_multilingual = property(lambda self: 0)
    cpu_backend = property(lambda self: "off")
    cpu_backend_note = property(lambda self: "this build has no CPU route; every input is encoded on the GPU")
    cpu_cost_model = property(lambda self: {})
    last_route = property(lambda self: "gpu")
    graph_capacities = property(lambda self: [self._cap])
    active_capacity = property(lambda self: self._cap)
    vocab_size = property(lambda self: int(self._g.lib.gtok_vocab_size(self._g.handle)))
    regex_kind = property(lambda self: _KINDS[self._g.family() & 0xFF])
    vocab_path = property(lambda self: self._path)


class Dispatcher:
    """Thread-safe front door shared by request threads (src/dispatcher.h, gtok_dispatch_*)."""

    def __init__(self, vocab_path, cpu_workers=1, max_batch_bytes=8 << 20, max_batch_docs=256, policy="adaptive", cpu_backend=""):
        if policy not in _POLICIES:
            raise ValueError("policy must be 'adaptive', 'gpu' or 'cpu'")
        if cpu_backend not in _BACKENDS:
            raise ValueError("cpu_backend must be one of '', 'auto', 'off', 'host', 'gigatoken'")
        self._lib = load_lib()
        self._workers = int(cpu_workers)
        self._h = self._lib.gtok_dispatcher_create(os.fsencode(os.fspath(vocab_path)), self._workers, int(max_batch_bytes), int(max_batch_docs),
                                                   _POLICIES[policy])
        if not self._h:
            raise GTokError("gtok_dispatcher_create failed: %s" % self._lib.gtok_x_last_error().decode("utf-8", "replace"))

    def encode_numpy(self, text):
        data = _as_bytes(text)
        out = np.empty(len(data) + 16, dtype=np.uint32)
        n = self._lib.gtok_dispatch_encode(self._h, data, len(data), out.ctypes.data, out.size)
        if n == -2:                                 # text its vocabulary's NFC lengthens
            out = np.empty(3 * len(data) + 64, dtype=np.uint32)
            n = self._lib.gtok_dispatch_encode(self._h, data, len(data), out.ctypes.data, out.size)
        if n < 0:
            raise RuntimeError("gtok_dispatch_encode returned %d" % n)
        return out[:n].copy()

    def stats(self):
        s = (ctypes.c_uint64 * 5)()
        self._lib.gtok_dispatcher_stats(self._h, s)
        return dict(zip(("cpu_requests", "gpu_requests", "gpu_batches", "gpu_large", "gpu_batch_ns"), (int(x) for x in s)))

    cpu_backend = property(lambda self: "off")
    cpu_workers = property(lambda self: self._workers)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.gtok_dispatcher_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
