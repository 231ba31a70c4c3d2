"""Seeded synthetic vocabularies and documents for the five benchmark configurations.

Everything is produced by the in-tree `datagen` tool from fixed seeds and cached
under `data_cache/` (or $GTOK_DATA_DIR); nothing is downloaded.  The real
vocabularies and corpora the reference was measured on are not available offline,
so these stand in for them with the stated shapes and value distributions.
"""
import hashlib
import os
import subprocess

import numpy as np

from . import build

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DATA_DIR = os.environ.get("GTOK_DATA_DIR", os.path.join(_ROOT, "data_cache"))

# name -> (family, corpus config, corpus seed, corpus bytes, merges, specials, corpus flags)
VOCABS = {
    "cfg0": ("gpt2", 0, 0, 32 << 20, 50000, 0, []),
    "cfg1": ("llama3", 1, 2, 32 << 20, 127744, 256, ["--no-specials"]),
    "cfg3": ("qwen25", 3, 5, 32 << 20, 151387, 22, ["--nfc"]),
    "cfg5": ("deepseek", 1, 9, 32 << 20, 100000, 16, ["--no-specials"]),
    # small vocabularies for quick tests
    "tiny_gpt2": ("gpt2", 0, 100, 2 << 20, 3000, 0, []),
    "tiny_llama3": ("llama3", 1, 101, 2 << 20, 4000, 8, ["--no-specials"]),
    "tiny_qwen25": ("qwen25", 3, 102, 2 << 20, 4000, 4, ["--nfc"]),
    "tiny_deepseek": ("deepseek", 1, 103, 2 << 20, 4000, 4, ["--no-specials"]),
}

# config id -> (vocab name, text config, seed, bytes)
DOCS = {
    0: ("cfg0", 0, 1, 4 << 20),
    1: ("cfg1", 1, 3, 4500000),
    3: ("cfg3", 3, 6, 8 << 20),
    4: ("cfg1", 4, 7, 32 << 20),
    5: ("cfg5", 1, 10, 4 << 20),      # beyond the five benchmark configurations: a DeepSeek-V3-shaped vocabulary
}
BATCH = ("cfg0", 4, 8192)   # config 2: vocab, seed, documents


def _run(args):
    subprocess.run([build.build_datagen()] + [str(a) for a in args], check=True, stderr=subprocess.DEVNULL)


def vocab_path(name):
    """Path of the tokenizer.json for a named synthetic vocabulary (trained on first use)."""
    os.makedirs(DATA_DIR, exist_ok=True)
    out = os.path.join(DATA_DIR, name + ".json")
    if os.path.exists(out):
        return out
    fam, cfg, seed, nbytes, merges, specials, flags = VOCABS[name]
    # (temporary names carry the process id: several ranks may generate the same file at once)
    corpus = os.path.join(DATA_DIR, "%s.corpus.%d.tmp" % (name, os.getpid()))
    _run(["text", cfg, seed, nbytes, corpus] + flags)
    tmp = "%s.%d.tmp" % (out, os.getpid())
    _run(["train", fam, corpus, merges, specials, tmp])
    os.replace(tmp, out)
    os.remove(corpus)
    return out


def text(config, seed, nbytes, flags=()):
    """Bytes of a synthetic document of the given text configuration."""
    os.makedirs(DATA_DIR, exist_ok=True)
    key = "text_%d_%d_%d%s.bin" % (config, seed, nbytes, "".join(flags))
    out = os.path.join(DATA_DIR, key)
    if not os.path.exists(out):
        tmp = "%s.%d.tmp" % (out, os.getpid())
        _run(["text", config, seed, nbytes, tmp] + list(flags))
        os.replace(tmp, out)
    with open(out, "rb") as f:
        return f.read()


def config_doc(config):
    """(tokenizer.json path, document bytes) for benchmark configuration 0, 1, 3 or 4 (5: DeepSeek-V3-shaped)."""
    vocab, tcfg, seed, nbytes = DOCS[config]
    return vocab_path(vocab), text(tcfg, seed, nbytes)


def config_batch(n_docs=None, seed=None):
    """(tokenizer.json path, blob, uint32 offsets) for the batch configuration (config 2)."""
    vocab, s, n = BATCH
    n_docs = n_docs or n
    seed = s if seed is None else seed
    os.makedirs(DATA_DIR, exist_ok=True)
    blob_p = os.path.join(DATA_DIR, "batch_%d_%d.bin" % (seed, n_docs))
    off_p = os.path.join(DATA_DIR, "batch_%d_%d.off" % (seed, n_docs))
    if not (os.path.exists(blob_p) and os.path.exists(off_p)):
        sfx = ".%d.tmp" % os.getpid()
        _run(["batch", seed, n_docs, blob_p + sfx, off_p + sfx])
        os.replace(off_p + sfx, off_p)
        os.replace(blob_p + sfx, blob_p)
    with open(blob_p, "rb") as f:
        blob = f.read()
    return vocab_path(vocab), blob, np.fromfile(off_p, dtype=np.uint32)


def sha256(data):
    return hashlib.sha256(data).hexdigest()
