"""CPU-side checks of the drop-in boundary and the host logic: exported symbols, the
tokenizer.json loader's acceptance rules, table construction, the shard planner and
a two-rank (gloo) run of the count exchange."""
import ctypes
import json
import os
import re
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from conftest import FAMILIES, ROOT, tiny_vocab
import oracle_lib


def test_library_exports_every_declared_symbol(built):
    import graphtok_b200
    header = open(os.path.join(ROOT, "include", "gtok.h")).read()
    declared = sorted(set(re.findall(r"\b(gtok_[a-z_0-9]+)\s*\(", header)))
    assert len(declared) >= 13
    lib = ctypes.CDLL(graphtok_b200.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", graphtok_b200.LIB_PATH], capture_output=True, text=True).stdout
    exported = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert exported and all(s.startswith("gtok_") for s in exported), exported
    for ref_name in ("gtok_create", "gtok_encode", "gtok_encode_to_device", "gtok_encode_batch", "gtok_cpu_max_bytes", "gtok_set_cpu_max_bytes",
                     "gtok_cpu_backend", "gtok_dispatcher_create", "gtok_dispatch_encode", "gtok_dispatcher_stats", "gtok_dispatcher_destroy",
                     "gtok_vocab_size", "gtok_destroy"):
        assert ref_name in exported


def test_no_cpu_route_and_loud_failure_without_gpu(built):
    import graphtok_b200
    lib = graphtok_b200.load_lib()
    assert lib.gtok_cpu_backend(None) == b"off"
    assert lib.gtok_cpu_max_bytes(None) == 0
    assert lib.gtok_create(b"/nonexistent/tokenizer.json", 4096) is None
    assert lib.gtok_encode(None, b"x", 1, None, 0) == -1
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        assert lib.gtok_create(os.fsencode(tiny_vocab("gpt2")), 4096) is None
        assert b"no CUDA device" in lib.gtok_x_last_error()
        with pytest.raises(graphtok_b200.GTokError):
            graphtok_b200.GTok(tiny_vocab("gpt2"))


def _mutate(family, fn):
    j = json.load(open(tiny_vocab(family)))
    fn(j)
    f = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(j, f)
    f.close()
    return f.name


def _loads(path):
    try:
        oracle_lib.Emul(path)
        return True
    except RuntimeError:
        return False


def test_loader_accepts_the_known_shapes_only(built):
    for f in FAMILIES:
        assert _loads(tiny_vocab(f))
    bad = [
        ("gpt2", lambda j: j["pre_tokenizer"].__setitem__("add_prefix_space", True)),
        ("gpt2", lambda j: j.__setitem__("normalizer", {"type": "NFC"})),
        ("llama3", lambda j: j["pre_tokenizer"]["pretokenizers"][0]["pattern"].__setitem__("Regex", "\\s+")),
        ("llama3", lambda j: j["model"].__setitem__("ignore_merges", False)),
        ("qwen25", lambda j: j.__setitem__("normalizer", None)),
        ("qwen25", lambda j: j["pre_tokenizer"]["pretokenizers"][1].__setitem__("trim_offsets", True)),
        ("gpt2", lambda j: j["model"].__setitem__("dropout", 0.1)),
        ("gpt2", lambda j: j["model"].__setitem__("byte_fallback", True)),
        ("gpt2", lambda j: j["model"].__setitem__("unk_token", "<unk>")),
        ("gpt2", lambda j: j["model"]["vocab"].pop("a")),
        ("gpt2", lambda j: j["model"]["merges"].append("zz qq")),
        ("llama3", lambda j: j["added_tokens"][0].__setitem__("lstrip", True)),
        ("llama3", lambda j: j["added_tokens"].append({"id": 999999, "content": "a<b", "special": True})),
        ("gpt2", lambda j: j["model"].__setitem__("type", "Unigram")),
        # DeepSeek-V3: an empty normalizer Sequence, the three exact Split patterns in their order, ByteLevel without its regex
        ("deepseek", lambda j: j.__setitem__("normalizer", None)),
        ("deepseek", lambda j: j["normalizer"]["normalizers"].append({"type": "NFC"})),
        ("deepseek", lambda j: j["pre_tokenizer"]["pretokenizers"].pop(1)),
        ("deepseek", lambda j: j["pre_tokenizer"]["pretokenizers"][0]["pattern"].__setitem__("Regex", "\\p{N}")),
        ("deepseek", lambda j: j["pre_tokenizer"]["pretokenizers"][2]["pattern"].__setitem__("Regex", j["pre_tokenizer"]["pretokenizers"][2]["pattern"]["Regex"].replace("[A-Za-z]+", "[a-z]+"))),
        ("deepseek", lambda j: j["pre_tokenizer"]["pretokenizers"][2].__setitem__("behavior", "Removed")),
        ("deepseek", lambda j: j["pre_tokenizer"]["pretokenizers"][3].__setitem__("use_regex", True)),
        ("deepseek", lambda j: j["model"].__setitem__("ignore_merges", True)),
        # Gemma-3: Replace " " by U+2581, the Split on " " merged with the previous piece, byte fallback with every "<0xNN>" token
        ("gemma", lambda j: j["normalizer"].__setitem__("content", "_")),
        ("gemma", lambda j: j["normalizer"]["pattern"].__setitem__("String", "  ")),
        ("gemma", lambda j: j.__setitem__("normalizer", None)),
        ("gemma", lambda j: j["pre_tokenizer"].__setitem__("behavior", "Isolated")),
        ("gemma", lambda j: j["pre_tokenizer"].__setitem__("invert", True)),
        ("gemma", lambda j: j["pre_tokenizer"]["pattern"].__setitem__("String", "\u2581")),
        ("gemma", lambda j: j["model"].__setitem__("byte_fallback", False)),
        ("gemma", lambda j: j["model"].__setitem__("fuse_unk", False)),
        ("gemma", lambda j: j["model"].__setitem__("unk_token", None)),
        ("gemma", lambda j: j["model"].__setitem__("ignore_merges", True)),
        ("gemma", lambda j: j["model"]["vocab"].pop("<0x7F>")),
        ("gemma", lambda j: j["model"]["vocab"].pop("\u2581")),
    ]
    for fam, fn in bad:
        p = _mutate(fam, fn)
        try:
            assert not _loads(p), fn
        finally:
            os.remove(p)
    with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
        f.write("{ not json")
    assert not _loads(f.name)
    os.remove(f.name)


def test_merges_as_pairs_are_accepted(built, oracles):
    def fn(j):
        j["model"]["merges"] = [m.split(" ") for m in j["model"]["merges"]]
    p = _mutate("gpt2", fn)
    try:
        e = oracle_lib.Emul(p)
        b = b"the quick brown fox"
        assert np.array_equal(e.encode(b), oracles["gpt2"].encode(b))
    finally:
        os.remove(p)


def test_added_token_matcher_agrees_with_the_oracle(built):
    """Added-token literals (path-compressed trie) against the oracle: literals that are prefixes of one
    another, that share stems, of many different lengths, next to each other and at tile edges."""
    import random
    rng = random.Random(9)

    def with_literals(lits):
        def fn(j):
            top = max(j["model"]["vocab"].values()) + 1
            j["added_tokens"] = [{"id": top + i, "content": c, "single_word": False, "lstrip": False, "rstrip": False,
                                  "normalized": False, "special": True} for i, c in enumerate(lits)]
        return fn

    # (the loader, like the reference's, refuses literals that contain a literal's first byte past their own start)
    few = ["<|a|>", "<|ab|>", "<|a", "<|abc|>x", "[x]", "[xy", "<|reserved_7|>", "<|reserved_77|>", "\u00a7\u00e9"]
    many = few + ["<" + "q" * k + ">" for k in range(1, 45)]
    for fam in ("llama3", "gpt2"):
        for lits in (few, many):
            path = _mutate(fam, with_literals(lits))
            try:
                o, e = oracle_lib.Oracle(path), oracle_lib.Emul(path)
                pool = lits + ["<|", "|>", "[", "<", "q", " word ", "x", "\n", "<|abc|", "\u00e9", "\u00a7", "7"]
                for it in range(300):
                    t = "".join(rng.choice(pool) for _ in range(rng.randint(1, 30)))
                    if it % 5 == 0:
                        t = "ab " * rng.randint(1300, 1400) + t + " tail"          # across a tile edge
                    if it == 7:
                        t = "[x]" * 1500 + t + "<|a|>" * 70 + "w"                 # far more literals than a tile's list holds
                    b = t.encode()
                    assert np.array_equal(e.encode(b, reverse=bool(it & 1)), o.encode_normalized(b)), (fam, len(lits), t[-80:])
            finally:
                os.remove(path)


def test_host_nfc_matches_unicodedata(built):
    """The library's NFC (used before the graph for Qwen2.5 vocabularies) against Python's, which
    Hugging Face's normaliser agrees with: named cases, a small-alphabet fuzz, every codepoint once."""
    import random
    import unicodedata as ud
    named = ["e\u0301", "a\u0308o\u0308", "A\u030a", "\u212b", "\u1e9b\u0323", "q\u0307\u0323", "\uac00", "\u1100\u1161\u11a8", "\u0958",
             "\u0b47\u0b56", "x\u0301\u0301\u0301", "\u0301a", "\ufb01 \u00bd \u2126", "a\u0323\u0302", "\u0f73", "\u1f71", "\u0344", "D\u0307\u0323",
             "\u09c7\u09be", "plain ascii", "", "\u65e5\u672c\u8a9e", "\U0001d15e", "\u0cc6\u0cc2\u0cd5"]
    for s in named:
        assert oracle_lib.lib_nfc(s.encode()) == ud.normalize("NFC", s).encode(), repr(s)
    rng = random.Random(4)
    pool = [chr(c) for c in list(range(0x41, 0x48)) + list(range(0x300, 0x370)) + [0xC0, 0xE9, 0x323, 0x1100, 0x1161, 0x11A8, 0xAC00, 0xAC01, 0x958, 0xB47,
                                                                                     0xB56, 0xB3E, 0x344, 0x340, 0x20, 0x3099, 0x304B, 0x1E0A, 0x1D157, 0x1D165]]
    for _ in range(20000):
        s = "".join(rng.choice(pool) for _ in range(rng.randint(1, 9)))
        assert oracle_lib.lib_nfc(s.encode()) == ud.normalize("NFC", s).encode(), [hex(ord(c)) for c in s]
    blob = "".join("a" + chr(cp) + "b" for cp in range(0x80, 0x30000) if not 0xD800 <= cp <= 0xDFFF)
    assert oracle_lib.lib_nfc(blob.encode()) == ud.normalize("NFC", blob).encode()
    # bytes that are not UTF-8 pass through untouched
    raw = b"ab\xcc\xff e\xcc\x81 \xe4\xb8"
    assert oracle_lib.lib_nfc(raw) == b"ab\xcc\xff \xc3\xa9 \xe4\xb8"


def test_document_plan_is_contiguous_and_balanced(built):
    import graphtok_b200
    rng = np.random.default_rng(0)
    lens = rng.integers(0, 5000, size=1000)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    for parts in (1, 2, 4, 8):
        cut = graphtok_b200.plan_documents(offs, parts)
        assert cut[0] == 0 and cut[-1] == 1000 and np.all(np.diff(cut.astype(np.int64)) >= 0)
        sizes = [int(offs[cut[k + 1]]) - int(offs[cut[k]]) for k in range(parts)]
        assert max(sizes) - min(sizes) <= 2 * 5000


WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
import numpy as np, torch, torch.distributed as dist
import oracle_lib, graphtok_b200
from graphtok_b200 import synth
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
path = synth.vocab_path("tiny_gpt2")
o = oracle_lib.Oracle(path)            # stands in for the per-GPU encoder in this CPU test
_, blob, offs = None, *synth.config_batch(64, seed=9)[1:]
cut = graphtok_b200.plan_documents(offs, world)
lo, hi = int(cut[rank]), int(cut[rank + 1])
ids, doc = o.encode_batch(blob, offs[lo:hi + 1])
counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
dist.all_gather(counts, torch.tensor([len(ids)], dtype=torch.int64))
base = int(sum(int(c) for c in counts[:rank]))
global_doc = doc.astype(np.int64) + base
gathered = [None] * world
dist.all_gather_object(gathered, (ids, global_doc))
if rank == 0:
    all_ids = np.concatenate([g[0] for g in gathered])
    all_doc = np.concatenate([g[1][:-1] for g in gathered] + [gathered[-1][1][-1:]])
    want_ids, want_doc = o.encode_batch(blob, offs)
    assert np.array_equal(all_ids, want_ids)
    assert np.array_equal(all_doc, want_doc.astype(np.int64))
# the other split: ONE document cut into one pre-token-aligned chunk per rank
import ctypes
lpath = synth.vocab_path("tiny_llama3")
lo_ = oracle_lib.Oracle(lpath)
e = oracle_lib.Emul(lpath)                # carries the library's planner (gtok_x_plan_chunks) without a GPU
text = synth.text(1, 5, 200000)
e.lib.gtok_emul_plan_chunks.restype = ctypes.c_int
e.lib.gtok_emul_plan_chunks.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p]
cuts = np.zeros(world + 1, dtype=np.uint64)
assert e.lib.gtok_emul_plan_chunks(e.h, text, len(text), world, cuts.ctypes.data) == 0
part_ids = lo_.encode_normalized(text[int(cuts[rank]):int(cuts[rank + 1])])
counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
dist.all_gather(counts, torch.tensor([len(part_ids)], dtype=torch.int64))
offsets = np.concatenate([[0], np.cumsum([int(c) for c in counts])])
gathered = [None] * world
dist.all_gather_object(gathered, part_ids)
if rank == 0:
    whole = lo_.encode_normalized(text)
    assert int(offsets[-1]) == len(whole) and np.array_equal(np.concatenate(gathered), whole)
    assert 0 < int(cuts[1]) < len(text)
    print("OK")
dist.destroy_process_group()
"""


def test_two_rank_document_sharding_with_gloo(built):
    """World size 2 on CPU, both ways the path shards: a batch by contiguous document ranges and one
    document by pre-token-aligned chunks; all-gather of token counts, global offsets, ids concatenated."""
    from graphtok_b200 import synth
    synth.config_batch(64, seed=9)      # generated once here, read by both ranks
    synth.vocab_path("tiny_llama3")
    synth.text(1, 5, 200000)
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER % {"root": ROOT})
    try:
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                            "--master-port", "29731", f.name], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    finally:
        os.remove(f.name)
