"""The kernels' tile programs, run serially on the CPU (tests/cpu_emul), against the oracle.
Covers the logic of pre-tokenization, the three merge paths, output assembly and the
per-document offsets without a GPU; the GPU tests repeat the comparison through the C ABI."""
import json
import os

import numpy as np
import pytest

import oracle_lib
from conftest import FAMILIES, GOLDEN, SPECIAL
import cases


def norm(o, b):
    return oracle_lib.nfc(b) if o.needs_nfc else b


def starts_without_dropped(starts, data):
    """Boundary bits on stray continuation bytes (dropped text at a document start) carry no pre-token."""
    return np.array([s for s in starts if (data[s] & 0xC0) != 0x80], dtype=np.uint32)


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_matches_golden(emuls, oracles, family):
    data = json.load(open(os.path.join(GOLDEN, "golden_%s.json" % family)))
    e, o = emuls[family], oracles[family]
    for row in data["cases"]:
        b = norm(o, row["text"].encode("utf-8"))
        assert e.encode(b).tolist() == row["ids"], repr(row["text"][:40])


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_fuzz_ids_and_boundaries(emuls, oracles, family):
    e, o = emuls[family], oracles[family]
    for i, t in enumerate(cases.fuzz_strings(21, SPECIAL[family], per_pool=220)):
        b = norm(o, t.encode())
        if not b:
            continue
        ids, st = e.encode(b, reverse=bool(i & 1), want_starts=True)
        want, wst = o.encode_normalized(b, want_starts=True)
        assert np.array_equal(ids, want), repr(t[:60])
        assert np.array_equal(starts_without_dropped(st, b), wst), repr(t[:60])


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_malformed_utf8(emuls, oracles, family):
    e, o = emuls[family], oracles[family]
    for b in cases.malformed_bytes(31, 400):
        assert np.array_equal(e.encode(b), o.encode_normalized(b)), repr(b)


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_tile_edges_and_long_runs(emuls, oracles, family):
    e, o = emuls[family], oracles[family]
    for i, t in enumerate(cases.tile_crossers(SPECIAL[family])):
        b = norm(o, t.encode())
        assert np.array_equal(e.encode(b, reverse=bool(i & 1)), o.encode_normalized(b)), (i, repr(t[-60:]))


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_length_ladder_all_merge_paths(emuls, oracles, family):
    e, o = emuls[family], oracles[family]
    for t in cases.length_ladder():
        b = t.encode()
        want = o.encode_normalized(b)
        assert np.array_equal(e.encode(b), want), (len(t), t[:20])
        # same answer from the one-merge-per-round path used for non-monotone vocabularies
        if len(b) <= 600:
            assert np.array_equal(e.encode(b, non_monotone=True), want), (len(t), t[:20])


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_batch_equals_per_document(emuls, oracles, family):
    e, o = emuls[family], oracles[family]
    docs = [norm(o, d.encode()) for d in cases.SEAM_DOCS] + [("word " * 900).encode(), b"\x80\x80abc", b"q" * 5000, ("7" * 4200).encode()]
    blob, offs = cases.make_batch(3, docs)
    ids, doc = e.encode(blob, offsets=offs)
    want_ids, want_doc = [], [0]
    for i in range(len(offs) - 1):
        t = o.encode_normalized(blob[int(offs[i]):int(offs[i + 1])])
        want_ids.append(t)
        want_doc.append(want_doc[-1] + len(t))
    assert np.array_equal(ids, np.concatenate(want_ids))
    assert doc.tolist() == want_doc


def test_emul_synthetic_documents(built):
    from graphtok_b200 import synth
    for name, cfg in (("tiny_gpt2", 0), ("tiny_llama3", 1), ("tiny_qwen25", 3), ("tiny_llama3", 4)):
        path = synth.vocab_path(name)
        e, o = oracle_lib.Emul(path), oracle_lib.Oracle(path)
        b = norm(o, synth.text(cfg, 77, 300000)[:260000].decode("utf-8", "ignore").encode())
        assert np.array_equal(e.encode(b), o.encode_normalized(b)), name


@pytest.mark.parametrize("family", ("gpt2", "llama3"))
def test_chunk_plan_concatenates(emuls, oracles, family):
    """Cutting a document at planned positions and encoding the parts gives the whole document's ids."""
    import ctypes
    from graphtok_b200 import synth
    e, o = emuls[family], oracles[family]
    doc = synth.text(1 if family == "llama3" else 0, 5, 200000)
    lib = e.lib
    lib.gtok_emul_plan_chunks.restype = ctypes.c_int
    lib.gtok_emul_plan_chunks.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p]
    for parts in (2, 3, 8):
        cuts = np.zeros(parts + 1, dtype=np.uint64)
        assert lib.gtok_emul_plan_chunks(e.h, doc, len(doc), parts, cuts.ctypes.data) == 0
        assert cuts[0] == 0 and cuts[-1] == len(doc) and np.all(np.diff(cuts.astype(np.int64)) >= 0)
        pieces = [o.encode_normalized(doc[int(cuts[k]):int(cuts[k + 1])]) for k in range(parts)]
        assert np.array_equal(np.concatenate(pieces), o.encode_normalized(doc))
