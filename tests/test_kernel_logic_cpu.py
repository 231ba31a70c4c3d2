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


def decoded(family, b):
    """What ids decode to when they were made from the bytes b: b itself, but for the Gemma-3 shape, whose U+2581 and
    space are one character of the vocabulary that decodes to a space."""
    return b.replace("\u2581".encode(), b" ") if family == "gemma" else b


def starts_without_dropped(starts, data, family=None):
    """Boundary bits on stray continuation bytes (dropped text at a document start) carry no pre-token -- except for the
    Gemma-3 shape, which spells every byte of the text."""
    if family == "gemma":
        return np.array(starts, dtype=np.uint32)
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
        assert np.array_equal(starts_without_dropped(st, b, family), wst), repr(t[:60])


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_added_tokens_by_trie_walk(emuls, oracles, family):
    """Literals are matched through a hash table when they have few distinct lengths and by a trie
    walk otherwise: the walk, forced here, gives the same ids."""
    e, o = emuls[family], oracles[family]
    if not SPECIAL[family]:
        pytest.skip("vocabulary without added tokens")
    for i, t in enumerate(cases.fuzz_strings(23, SPECIAL[family], per_pool=60)):
        b = norm(o, t.encode())
        if b:
            assert np.array_equal(e.encode(b, trie=True, reverse=bool(i & 1)), o.encode_normalized(b)), repr(t[:60])


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
    for name, cfg in (("tiny_gpt2", 0), ("tiny_llama3", 1), ("tiny_qwen25", 3), ("tiny_llama3", 4), ("tiny_deepseek", 1), ("tiny_deepseek", 4), ("tiny_deepseek", 3)):
        path = synth.vocab_path(name)
        e, o = oracle_lib.Emul(path), oracle_lib.Oracle(path)
        b = norm(o, synth.text(cfg, 77, 300000)[:260000].decode("utf-8", "ignore").encode())
        assert np.array_equal(e.encode(b), o.encode_normalized(b)), name


@pytest.mark.parametrize("family", ("gpt2", "llama3", "deepseek"))
def test_chunk_plan_concatenates(emuls, oracles, family):
    """Cutting a document at planned positions and encoding the parts gives the whole document's ids."""
    import ctypes
    from graphtok_b200 import synth
    e, o = emuls[family], oracles[family]
    doc = synth.text(0 if family == "gpt2" else 1, 5, 200000)
    lib = e.lib
    lib.gtok_emul_plan_chunks.restype = ctypes.c_int
    lib.gtok_emul_plan_chunks.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p]
    for parts in (2, 3, 8):
        cuts = np.zeros(parts + 1, dtype=np.uint64)
        assert lib.gtok_emul_plan_chunks(e.h, doc, len(doc), parts, cuts.ctypes.data) == 0
        assert cuts[0] == 0 and cuts[-1] == len(doc) and np.all(np.diff(cuts.astype(np.int64)) >= 0)
        pieces = [o.encode_normalized(doc[int(cuts[k]):int(cuts[k + 1])]) for k in range(parts)]
        assert np.array_equal(np.concatenate(pieces), o.encode_normalized(doc))


def _nfc_pool():
    marks = [0x300, 0x301, 0x302, 0x308, 0x323, 0x327, 0x31B, 0x345, 0x334, 0x340, 0x341, 0x343, 0x344, 0x5B4, 0x64B, 0x651, 0x93C, 0x94D, 0x9BE, 0x9D7,
             0xB3E, 0xB56, 0xB57, 0xBBE, 0xCC2, 0xCD5, 0xD3E, 0xDCA, 0xDCF, 0xF71, 0xF72, 0xF74, 0x102E, 0x1161, 0x1175, 0x11A8, 0x11C2, 0x1B35, 0x3099,
             0x309A, 0x1D165, 0x1D16E, 0x110BA, 0x11127, 0x1133E, 0x114B0, 0x115AF, 0x11930]
    bases = [ord(c) for c in "aeiouAEONcy =\n1."] + [0xE9, 0x1EA0, 0x1100, 0x1112, 0xAC00, 0xAC01, 0xD55C, 0x915, 0x9C7, 0xB47, 0xBC6, 0xCC6, 0xD46, 0xDD9,
             0xF40, 0x1025, 0x1B05, 0x3046, 0x304B, 0x4E2D, 0x2126, 0x212B, 0xF900, 0xFB1D, 0xFB2A, 0x2000, 0x958, 0xFA30, 0x1D15E, 0x2F800, 0x1F600,
             0x11099, 0x11131, 0x11347, 0x114B9, 0x115B8, 0x11935, 0x1E69, 0x3A9, 0x438, 0x5E9, 0x644, 0x1F80]
    return marks, bases


def test_device_normaliser_matches_unicodedata_and_host():
    """The NFC tile program (csrc/nfc_core.h) on the CPU emulation, both thread orders, against Python's
    unicodedata (well-formed text) and the library's host normaliser (any bytes)."""
    import random
    import unicodedata as ud
    rng = random.Random(11)
    marks, bases = _nfc_pool()

    def rand_text(k):
        out = []
        for _ in range(k):
            r = rng.random()
            out.append(chr(rng.choice(bases)) if r < 0.5 else chr(rng.choice(marks)) if r < 0.9 else
                       chr(rng.choice(bases)) * rng.randint(1, 20) if r < 0.95 else "plain words " * rng.randint(0, 3))
        return "".join(out)

    named = ["e\u0301", "\u212b", "\u1100\u1161\u11a8", "\u0958", "x\u0301\u0301\u0301", "\u0301a", "a\u0323\u0302", "\u0344", "", "ascii only",
             "\u65e5\u672c\u8a9e", "\U0001d15e", "a" * 4095 + "\u0301", "a" * 4094 + "e\u0301", "e\u0301" * 3000, "\uac00\u11a8" * 2000]
    for s in named:
        for rev in (False, True):
            assert oracle_lib.device_nfc(s.encode(), reverse=rev) == ud.normalize("NFC", s).encode(), repr(s[:20])
    for it in range(250):
        s = rand_text(rng.randint(0, 60) if it % 5 else rng.randint(500, 2500))
        b = s.encode()
        assert oracle_lib.device_nfc(b, reverse=bool(it & 1)) == ud.normalize("NFC", s).encode(), it
        if it % 4 == 1 and b:      # the same with some bytes broken: the host normaliser defines the result
            bl = bytearray(b)
            for _ in range(rng.randint(1, 6)):
                bl[rng.randrange(len(bl))] = rng.choice([0x80, 0xBF, 0xC0, 0xC3, 0xE2, 0xF0, 0xFF, 0xCC, 0x41])
            assert oracle_lib.device_nfc(bytes(bl), reverse=bool(it & 2)) == oracle_lib.lib_nfc(bytes(bl)), it
    blob = "".join("a" + chr(cp) + "b" for cp in range(0x80, 0x30000) if not 0xD800 <= cp <= 0xDFFF)
    assert oracle_lib.device_nfc(blob.encode()) == ud.normalize("NFC", blob).encode()


def test_device_normaliser_batches_documents_apart():
    """Documents are normalised one by one (a mark at the start of one does not combine with the end of the
    one before, a codepoint cut by a document boundary is left alone) and their offsets are rewritten."""
    import random
    rng = random.Random(12)
    marks, bases = _nfc_pool()
    for it in range(150):
        s = "".join(chr(rng.choice(bases if rng.random() < 0.5 else marks)) for _ in range(rng.randint(1, 400)))
        b = s.encode()
        offs = [0] + sorted(rng.randrange(len(b) + 1) for _ in range(rng.randint(0, 7))) + [len(b)]
        if it % 3 == 0:
            offs.append(len(b))
        want, want_offs = b"", [0]
        for i in range(len(offs) - 1):
            want += oracle_lib.lib_nfc(b[offs[i]:offs[i + 1]])
            want_offs.append(len(want))
        got = oracle_lib.device_nfc(b, doc_off=offs, reverse=bool(it & 1))
        assert got == (want, want_offs), (it, offs)


def test_device_normaliser_reports_what_it_cannot_do():
    """A stretch of more codepoints than one thread takes and a result longer than the buffer set error
    bits (the engine then normalises on the host, or retries with a larger buffer); text flagged as
    normalised already is copied as it is."""
    zalgo = ("a" + "\u0301\u0323" * 60).encode()
    assert oracle_lib.device_nfc(zalgo) == -16
    assert oracle_lib.device_nfc(zalgo, already_normalised=True) == zalgo
    grows = ("\u0958 " * 100).encode()
    assert oracle_lib.device_nfc(grows, cap=len(grows) + 10) == -32
    assert oracle_lib.device_nfc(grows) == oracle_lib.nfc(grows)


@pytest.mark.parametrize("family", FAMILIES)
def test_emul_decode_against_the_vocabulary_file_and_round_trip(emuls, oracles, family):
    """decode_tile: random ids against a join of the spellings read from the tokenizer.json; the
    golden texts back from their ids; encode -> decode round trips over several tiles."""
    from conftest import tiny_vocab
    e, o = emuls[family], oracles[family]
    table = oracle_lib.token_spellings(tiny_vocab(family))
    known = np.array(sorted(table), dtype=np.uint32)
    rng = np.random.default_rng(5)
    for i, n in enumerate((1, 7, 8, 9, 255, 2047, 2048, 2049, 5000, 12345)):
        ids = rng.choice(known, size=n)
        want = b"".join(table[int(t)] for t in ids)
        got, total, bits = e.decode(ids, reverse=bool(i & 1))
        assert bits == 0 and total == len(want) and got == want, n
    data = json.load(open(os.path.join(GOLDEN, "golden_%s.json" % family)))
    for row in data["cases"]:
        got, _, bits = e.decode(row["ids"])
        assert bits == 0 and got == decoded(family, norm(o, row["text"].encode("utf-8"))), repr(row["text"][:40])
    for t in list(cases.fuzz_strings(77, SPECIAL[family], per_pool=25)) + [("naïve café — 日本語 " * 900)]:
        b = norm(o, t.encode())
        ids = o.encode_normalized(b)
        got, _, bits = e.decode(ids)
        assert bits == 0 and got == decoded(family, b), repr(t[:40])
    # one long token repeated: several rounds of the staging buffer per tile
    longest = max(table, key=lambda t: len(table[t]))
    ids = np.full(6000, longest, dtype=np.uint32)
    got, total, bits = e.decode(ids, cap=len(table[longest]) * 6000 + 3)
    assert bits == 0 and got == table[longest] * 6000


def test_emul_decode_errors(emuls):
    e = emuls["llama3"]
    from conftest import tiny_vocab
    table = oracle_lib.token_spellings(tiny_vocab("llama3"))
    ids = np.array(sorted(table)[:3000], dtype=np.uint32)
    want = b"".join(table[int(t)] for t in ids)
    got, total, bits = e.decode(ids, cap=len(want) - 1)            # too small: the count is still reported
    assert got is None and total == len(want) and bits & 1
    got, total, bits = e.decode(ids, cap=len(want))                 # exact fit
    assert got == want and bits == 0
    got, total, bits = e.decode(np.array([1, 2, 0x7FFFFFFF, 3], dtype=np.uint32))
    assert bits & 64                                                # an id outside the vocabulary
    got, total, bits = e.decode(np.zeros(0, dtype=np.uint32))
    assert total == 0 and bits == 0


def test_window_bit_scans_against_plain_loops(built):
    """plain_ws_end / newline_run_begin (csrc/encode_core.h): the first byte at or after i that is not plain one-byte
    whitespace of the running document, and the first of the newline bytes that end at i, from the bit planes --
    against byte-by-byte loops over the same bits, on random planes with long clean stretches, from every kind of
    start position and bound."""
    import ctypes, random
    lib = ctypes.CDLL(oracle_lib.build_emul())
    lib.gtok_emul_plain_ws_end.restype = ctypes.c_int
    lib.gtok_emul_plain_ws_end.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int, ctypes.c_int]
    lib.gtok_emul_newline_run_begin.restype = ctypes.c_int
    lib.gtok_emul_newline_run_begin.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_int, ctypes.c_int]
    rng = random.Random(77)
    n = 8192
    for trial in range(60):
        # whitespace / newline / document-start bits per byte: mostly long clean stretches with a few breaks
        density = rng.choice((0.0, 0.0005, 0.003, 0.02, 0.3))
        ws = np.ones(n, dtype=bool)
        cr = np.zeros(n, dtype=bool)
        doc = np.zeros(n, dtype=bool)
        for arr, val in ((ws, False), (cr, True), (doc, True)):
            for _ in range(int(n * density) + rng.randint(0, 2)):
                arr[rng.randrange(n)] = val
        if trial % 3 == 0:
            cr[:] = ~cr                                           # newline stretches for the backward scan
        pack16 = lambda b: np.packbits(b.reshape(-1, 16), axis=1, bitorder="little").view(np.uint16).reshape(-1)
        pack32 = lambda b: np.packbits(b.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).reshape(-1)
        s16 = np.concatenate([pack16(ws), np.zeros(8, np.uint16)])
        c16 = np.concatenate([pack16(cr), np.zeros(8, np.uint16)])
        d32 = np.concatenate([pack32(doc), np.zeros(4, np.uint32)])
        good_f = ws & ~cr & ~doc
        good_b = cr & ~doc
        for _ in range(200):
            i = rng.choice((rng.randrange(n), rng.randrange(n) & ~63, (rng.randrange(n) & ~63) | 63, 0, n - 1))
            i_end = rng.choice((n, rng.randrange(n + 1), min(n, i + rng.randrange(600))))
            want = i_end
            if i < i_end:
                bad = np.flatnonzero(~good_f[i:i_end])
                if bad.size: want = i + int(bad[0])
            assert lib.gtok_emul_plain_ws_end(s16.ctypes.data, c16.ctypes.data, d32.ctypes.data, i, i_end) == want, (trial, i, i_end)
            i_begin = rng.choice((0, rng.randrange(n), max(0, i - rng.randrange(600))))
            if i < i_begin:
                want_b = i + 1
            else:
                bad = np.flatnonzero(~good_b[i_begin:i + 1])
                want_b = i_begin if not bad.size else i_begin + int(bad[-1]) + 1
            assert lib.gtok_emul_newline_run_begin(c16.ctypes.data, d32.ctypes.data, i, i_begin) == want_b, (trial, i, i_begin)


def test_normaliser_table_lookups_cover_every_codepoint_and_pair(built):
    """The device side finds a codepoint's combining class and decomposition, and a pair's composite, in hashed
    tables (csrc/nfc_core.h: nfc_cp_info, nfc_compose).  Every codepoint and every composing pair against
    Python's unicodedata, and pairs that do not compose."""
    import ctypes, random, unicodedata
    lib = ctypes.CDLL(oracle_lib.build_emul())
    n = 0x110000
    info = np.zeros(n, dtype=np.uint32)
    lib.gtok_emul_nfc_cp_info(ctypes.c_void_p(info.ctypes.data), ctypes.c_uint32(n))
    firsts, seconds, wants = [], [], []
    for cp in range(n):
        if 0xD800 <= cp <= 0xDFFF:
            continue
        ch = chr(cp)
        assert (info[cp] & 0xFF) == unicodedata.combining(ch), hex(cp)
        hangul = 0xAC00 <= cp < 0xAC00 + 11172
        full = unicodedata.normalize("NFD", ch)
        if not hangul:                                            # Hangul syllables are decomposed by arithmetic, not from the table
            assert (info[cp] >> 8) == (len(full) if full != ch else 0), hex(cp)
        dec = unicodedata.decomposition(ch)
        if dec and not dec.startswith("<") and len(dec.split()) == 2:
            a, b = (int(x, 16) for x in dec.split())
            back = unicodedata.normalize("NFC", chr(a) + chr(b))
            firsts.append(a); seconds.append(b); wants.append(ord(back) if len(back) == 1 else 0)
    rng = random.Random(5)
    pool = sorted(set(firsts) | set(seconds))
    for _ in range(20000):                                        # other pairs of the same codepoints: whatever NFC says
        a, b = rng.choice(pool), rng.choice(pool)
        back = unicodedata.normalize("NFC", chr(a) + chr(b))
        if unicodedata.normalize("NFD", chr(a)) != chr(a) or unicodedata.normalize("NFD", chr(b)) != chr(b):
            continue                                              # (the kernel composes decomposed input only)
        firsts.append(a); seconds.append(b); wants.append(ord(back) if len(back) == 1 else 0)
    f = np.array(firsts, dtype=np.uint32); s2 = np.array(seconds, dtype=np.uint32); out = np.zeros(len(firsts), dtype=np.uint32)
    lib.gtok_emul_nfc_compose(ctypes.c_void_p(f.ctypes.data), ctypes.c_void_p(s2.ctypes.data), ctypes.c_void_p(out.ctypes.data), ctypes.c_uint32(len(firsts)))
    bad = np.flatnonzero(out != np.array(wants, dtype=np.uint32))
    assert bad.size == 0, [(hex(firsts[i]), hex(seconds[i]), hex(int(out[i])), hex(wants[i])) for i in bad[:5]]
