"""Parity proper: libgtok on a B200, called through its C ABI, against the oracle and the
golden vectors.  Ids are integers: every comparison is exact."""
import ctypes
import json
import os
import threading

import numpy as np
import pytest

import oracle_lib
from conftest import FAMILIES, GOLDEN, SPECIAL, tiny_vocab
import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gtoks(built):
    from graphtok_b200 import GTok
    hs = {f: GTok(tiny_vocab(f), max_bytes=1 << 20) for f in FAMILIES}
    yield hs
    for h in hs.values():
        h.close()


def norm(o, b):
    return oracle_lib.nfc(b) if o.needs_nfc else b


@pytest.mark.parametrize("family", FAMILIES)
def test_golden_vectors(gtoks, oracles, family):
    data = json.load(open(os.path.join(GOLDEN, "golden_%s.json" % family)))
    g, o = gtoks[family], oracles[family]
    for row in data["cases"]:
        b = norm(o, row["text"].encode("utf-8"))
        assert g.encode(b).tolist() == row["ids"], repr(row["text"][:40])


@pytest.mark.parametrize("family", FAMILIES)
def test_fuzz_malformed_edges_and_lengths(gtoks, oracles, family):
    g, o = gtoks[family], oracles[family]
    texts = [t.encode() for t in cases.fuzz_strings(41, SPECIAL[family], per_pool=150)]
    texts += cases.malformed_bytes(43, 200)
    texts += [t.encode() for t in cases.tile_crossers(SPECIAL[family])]
    texts += [t.encode() for t in cases.length_ladder()]
    for b in texts:
        b = norm(o, b) if b.decode("utf-8", "ignore").encode() == b else b
        assert np.array_equal(g.encode(b), o.encode_normalized(b)), repr(b[:60])


@pytest.mark.parametrize("family", ("gpt2", "llama3"))
def test_short_inputs_without_the_one_kernel_graph(built, oracles, family):
    """Single documents of up to 2,048 bytes normally run as one single-block kernel; with that route
    switched off (GTOK_TINY=0) the four-kernel graph must give the same ids on the same short inputs."""
    from graphtok_b200 import GTok
    o = oracles[family]
    os.environ["GTOK_TINY"] = "0"
    try:
        g = GTok(tiny_vocab(family), max_bytes=1 << 20)
    finally:
        del os.environ["GTOK_TINY"]
    try:
        texts = [t.encode() for t in cases.fuzz_strings(45, SPECIAL[family], per_pool=80)] + cases.malformed_bytes(47, 100)
        texts += [t.encode() for t in cases.length_ladder()]
        for b in texts:
            assert np.array_equal(g.encode(b), o.encode_normalized(b)), repr(b[:60])
    finally:
        g.close()


def test_one_kernel_graph_sizes_and_return_codes(gtoks, oracles):
    """The single-block route at and around its size limit, on a handle that alternates with long inputs,
    and its -2 answer when the caller's buffer is too small."""
    from graphtok_b200 import synth
    g, o = gtoks["llama3"], oracles["llama3"]
    doc = synth.text(1, 77, 300000)
    for n in (1, 15, 16, 17, 2047, 2048, 2049, 4095, 4096, 4097, 8000, 8001, 12000, 3, 2048, 200000, 64):
        b = doc[:n].decode("utf-8", "ignore").encode()
        assert np.array_equal(g.encode(b), o.encode_normalized(b)), n
    b = doc[:5000].decode("utf-8", "ignore").encode()
    small = np.zeros(8, dtype=np.uint32)
    assert g.lib.gtok_encode(g.handle, b, len(b), small.ctypes.data, small.size) == -2
    assert np.array_equal(g.encode(b), o.encode_normalized(b))


@pytest.mark.parametrize("family", FAMILIES)
def test_batch_equals_per_document(gtoks, oracles, family):
    g, o = gtoks[family], oracles[family]
    docs = [norm(o, d.encode()) for d in cases.SEAM_DOCS] + [("word " * 900).encode(), b"\x80\x80abc", b"q" * 5000, ("7" * 4200).encode()]
    blob, offs = cases.make_batch(3, docs)
    ids, doc = g.encode_batch(blob, offs)
    want_ids, want_doc = [], [0]
    for i in range(len(offs) - 1):
        t = o.encode_normalized(blob[int(offs[i]):int(offs[i + 1])])
        want_ids.append(t)
        want_doc.append(want_doc[-1] + len(t))
    assert np.array_equal(ids, np.concatenate(want_ids))
    assert doc.tolist() == want_doc
    # the same handle keeps answering single documents identically afterwards
    assert np.array_equal(g.encode(b"after the batch"), o.encode_normalized(b"after the batch"))


@pytest.mark.parametrize("family", FAMILIES)
def test_boundary_bits_match_oracle_starts(gtoks, oracles, family):
    g, o = gtoks[family], oracles[family]
    for t in cases.fuzz_strings(51, SPECIAL[family], per_pool=40) + cases.tile_crossers(SPECIAL[family])[:30]:
        b = norm(o, t.encode())
        if not b:
            continue
        g.stage(b)
        g.replay()
        _, want = o.encode_normalized(b, want_starts=True)
        assert np.array_equal(g.boundaries(len(b)), want), repr(t[:60])


def test_qwen_raw_text_is_normalised_inside_the_call(gtoks, oracles):
    """gtok_encode applies the vocabulary's NFC itself: raw (decomposed) text gives the golden ids."""
    data = json.load(open(os.path.join(GOLDEN, "golden_qwen25.json")))
    g = gtoks["qwen25"]
    for row in data["cases"]:
        assert g.encode(row["text"].encode("utf-8")).tolist() == row["ids"], repr(row["text"][:40])
    docs = ["cafe\u0301", "", "nai\u0308ve", "plain", "\u1100\u1161\u11a8 x"]
    blob, offs = cases.make_batch(5, docs)
    ids, doc = g.encode_batch(blob, offs)
    want, want_doc = oracles["qwen25"].encode_batch(blob, offs)
    assert np.array_equal(ids, want) and np.array_equal(doc, want_doc)


def test_qwen_normalisation_on_the_device_large_and_odd_cases(oracles):
    """NFC runs as the graph's first kernel: decomposed text over many tiles, a batch whose documents cut
    codepoints, a stretch too long for a thread (host normalisation, then a copy-only pass), text that NFC
    lengthens past the context (rebuilt larger), and the byte cap applying to the normalised length."""
    import unicodedata as ud
    from graphtok_b200 import GTok
    o = oracles["qwen25"]
    g = GTok(tiny_vocab("qwen25"), max_bytes=1 << 16)
    try:
        base = "Vi\u1ec7t Nam c\u00f3 nhi\u1ec1u \ud55c\uad6d\uc5b4 na\u00efve caf\u00e9 \u65e5\u672c "
        nfd = ud.normalize("NFD", base * 1000).encode()
        assert len(nfd) > (1 << 16) >= len(ud.normalize("NFC", base * 1000).encode())      # raw over the cap, normalised under it
        assert np.array_equal(g.encode(nfd), o.encode(nfd))
        assert np.array_equal(g.encode(nfd), o.encode(nfd))
        zalgo = ("z" + "\u0301\u0323\u0308" * 50 + " ok ").encode() * 3
        assert np.array_equal(g.encode(zalgo), o.encode(zalgo))
        docs = [ud.normalize("NFD", base * 3), "\u0301x", "", "e", "\u0301\u0323", zalgo.decode(), "tail e\u0301"]
        blob, offs = cases.make_batch(9, docs)
        ids, doc = g.encode_batch(blob, offs)
        want, want_doc = o.encode_batch(blob, offs)
        assert np.array_equal(ids, want) and np.array_equal(doc, want_doc)
        raw = ud.normalize("NFD", base * 40).encode()
        cuts = [0, 5, 6, 7, 100, 101, 1000, 1001, 1002, len(raw) // 2, len(raw)]
        ids, doc = g.encode_batch(raw, np.array(cuts, dtype=np.uint32))
        parts = [o.encode_normalized(oracle_lib.lib_nfc(raw[cuts[i]:cuts[i + 1]])) for i in range(len(cuts) - 1)]
        assert np.array_equal(ids, np.concatenate(parts)) and doc.tolist() == np.cumsum([0] + [len(x) for x in parts]).tolist()
    finally:
        g.close()
    small = GTok(tiny_vocab("qwen25"), max_bytes=4096)
    try:
        grows = ("\u0958 " * 1000).encode()                  # 4000 bytes that become 7000
        out = np.zeros(8192, dtype=np.uint32)
        assert small.lib.gtok_encode(small.handle, grows, len(grows), out.ctypes.data, out.size) == -3
        ok = ("\u0958 " * 500).encode()                      # 2000 bytes that become 3500
        assert np.array_equal(small.encode(ok), o.encode(ok))
    finally:
        small.close()


def test_return_codes(gtoks):
    g = gtoks["gpt2"]
    lib = g.lib
    out = np.zeros(4, dtype=np.uint32)
    text = b"many words in a row " * 50
    assert lib.gtok_encode(g.handle, text, len(text), out.ctypes.data, 4) == -2
    big = b"x" * ((1 << 20) + 1)
    assert lib.gtok_encode(g.handle, big, len(big), out.ctypes.data, 4) == -3
    assert lib.gtok_encode(g.handle, b"", 0, out.ctypes.data, 4) == 0
    assert lib.gtok_encode(None, b"a", 1, out.ctypes.data, 4) == -1
    offs = np.array([0, 3, 2], dtype=np.uint32)
    doc = np.zeros(3, dtype=np.uint32)
    assert lib.gtok_encode_batch(g.handle, b"abcd", offs.ctypes.data, 2, out.ctypes.data, 4, doc.ctypes.data) == -1
    assert lib.gtok_vocab_size(g.handle) > 256
    assert lib.gtok_cpu_backend(g.handle) == b"off"
    # a failed call leaves the handle usable
    assert g.encode(b"still fine").size > 0


def test_encode_to_device_matches_host(gtoks, oracles):
    import torch
    g, o = gtoks["llama3"], oracles["llama3"]
    text = ("device side output " * 200).encode()
    buf = torch.zeros(len(text), dtype=torch.int32, device="cuda")
    n = g.lib.gtok_encode_to_device(g.handle, text, len(text), ctypes.c_void_p(buf.data_ptr()), buf.numel())
    assert n > 0
    torch.cuda.synchronize()
    assert np.array_equal(buf[:n].cpu().numpy().astype(np.uint32), o.encode_normalized(text))


def test_page_locked_output_buffer_is_written_directly(gtoks, oracles):
    """A caller's page-locked buffer receives the ids without the staging copy: same ids as through a
    pageable one, for a single document and for a batch (ids direct, document offsets staged)."""
    import torch
    g, o = gtoks["llama3"], oracles["llama3"]
    text = ("page locked output, many ids to copy. " * 25000).encode()          # > 512 KB of ids, under the handle's 1 MiB
    want = o.encode_normalized(text)
    pinned = torch.zeros(len(text) + 16, dtype=torch.int32).pin_memory()
    arr = pinned.numpy()
    n = g.lib.gtok_encode(g.handle, text, len(text), arr.ctypes.data, arr.size)
    assert n == len(want) and np.array_equal(arr[:n].view(np.uint32), want)
    offs = np.array([0, 5, 5, len(text) // 2, len(text)], dtype=np.uint32)
    docs = np.zeros(offs.size, dtype=np.uint32)
    arr[:] = 0
    n = g.lib.gtok_encode_batch(g.handle, text, offs.ctypes.data, offs.size - 1, arr.ctypes.data, arr.size, docs.ctypes.data)
    want_ids, want_doc = o.encode_batch(text, offs)
    assert n == len(want_ids) and np.array_equal(arr[:n].view(np.uint32), want_ids) and np.array_equal(docs, want_doc)


def test_sizes_change_between_calls_on_one_handle(gtoks, oracles):
    g, o = gtoks["llama3"], oracles["llama3"]
    from graphtok_b200 import synth
    doc = synth.text(4, 5, 900000)
    for n in (900000, 17, 4096, 300000, 1, 4097, 65536, 899999, 5):
        b = doc[:n].decode("utf-8", "ignore").encode()
        assert np.array_equal(g.encode(b), o.encode_normalized(b)), n


@pytest.mark.parametrize("policy", ("adaptive", "gpu", "cpu"))
def test_dispatcher_threads(built, oracles, policy):
    """Sixteen request threads against one dispatcher, 300 requests of 0 to 120,000 bytes, every
    policy name the reference accepts (the shape of its tests/test_dispatcher.py:37-81): every answer
    equals the oracle's, every request is counted once, and replays are shared (fewer batch replays
    than requests answered from them)."""
    import random
    import gpu_bpe_tokenizer
    from graphtok_b200 import synth
    corpus = synth.text(1, 77, 300000).decode("utf-8", "ignore")
    rng = random.Random(len(policy))
    items = []
    for _ in range(300):
        size = rng.choice((0, 1, 40, 700, 3000, 9000, 30000, 120000))
        a = rng.randrange(0, max(1, len(corpus) - size))
        items.append(corpus[a:a + size])
    items += ["<|reserved_special_token_3|>hi<|reserved_special_token_1|>", "\u00e9 x}\nfoo 1234567"]
    o = oracles["llama3"]
    d = gpu_bpe_tokenizer.Dispatcher(tiny_vocab("llama3"), cpu_workers=2, max_batch_bytes=1 << 20, max_batch_docs=64, policy=policy)
    results = [None] * len(items)
    idx = iter(range(len(items)))
    lock = threading.Lock()
    start = threading.Barrier(16)

    def worker():
        start.wait()
        while True:
            with lock:
                i = next(idx, None)
            if i is None:
                return
            results[i] = d.encode_numpy(items[i])

    ts = [threading.Thread(target=worker) for _ in range(16)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for i, (text, ids) in enumerate(zip(items, results)):
        assert ids is not None and np.array_equal(ids, o.encode(text.encode("utf-8"))), "request %d (%d chars) differs" % (i, len(text))
    s = d.stats()
    d.close()
    assert s["cpu_requests"] == 0                       # no CPU route in this library, whatever the policy
    assert s["cpu_requests"] + s["gpu_requests"] + s["gpu_large"] == len(items)
    assert s["gpu_batches"] < s["gpu_requests"]         # sixteen threads against one batcher must share replays


@pytest.mark.parametrize("config", (0, 1, 3, 5))
def test_benchmark_configurations_full_size(built, config):
    """Configurations 0, 1 and 3 at their full sizes against the oracle (5: the DeepSeek-V3-shaped vocabulary on 4 MiB)."""
    from graphtok_b200 import GTok, synth
    path, doc = synth.config_doc(config)
    o = oracle_lib.Oracle(path)
    b = norm(o, doc)
    want = o.encode_normalized(b)
    g = GTok(path, max_bytes=len(b) + 4096)
    try:
        assert np.array_equal(g.encode(b), want)
        if o.needs_nfc:
            assert np.array_equal(g.encode(doc), want)          # the raw document: the graph normalises it
    finally:
        g.close()
    # a page-locked input buffer is read by the device directly (no staging copy): same ids
    import torch
    pinned = torch.frombuffer(bytearray(doc), dtype=torch.uint8).pin_memory()
    out = np.empty(3 * len(doc) + 64, dtype=np.uint32)
    g2 = GTok(path, max_bytes=len(b) + 4096)
    try:
        n = g2.lib.gtok_encode(g2.handle, ctypes.c_void_p(pinned.data_ptr()), len(doc), out.ctypes.data, out.size)
        assert n == want.size and np.array_equal(out[:n], want)
    finally:
        g2.close()
    # the same with the staging copies on the calling thread alone
    os.environ["GTOK_COPY_THREADS"] = "1"
    try:
        g1 = GTok(path, max_bytes=len(b) + 4096)
        try:
            assert np.array_equal(g1.encode(doc), want)
        finally:
            g1.close()
    finally:
        del os.environ["GTOK_COPY_THREADS"]


def _reference_or_none(path):
    """The reference's own host encoder (oracle/_ref, built from its sources) when it is there."""
    if os.path.exists(oracle_lib.REF_SO):
        return oracle_lib.Reference(path)
    return None


def test_configuration_4_full_size_and_chunks(built):
    """Adversarial document at its stated 32 MB: the ids of one replay against the oracle (and the
    reference's own encoder when it was built), and the concatenation of eight planned chunks
    against the same ids."""
    from graphtok_b200 import GTok, synth
    path, doc = synth.config_doc(4)
    want = oracle_lib.Oracle(path).encode_normalized(doc)
    ref = _reference_or_none(path)
    if ref is not None:
        assert np.array_equal(ref.encode_normalized(doc), want)
    g = GTok(path, max_bytes=len(doc) + 4096)
    try:
        assert np.array_equal(g.encode(doc), want)
        cuts = g.plan_chunks(doc, 8)
        parts = [g.encode(doc[int(cuts[k]):int(cuts[k + 1])]) for k in range(8)]
        assert np.array_equal(np.concatenate(parts), want)
    finally:
        g.close()


def test_deepseek_vocabulary_on_the_adversarial_document(built):
    """The 32 MB adversarial document (long runs of one whitespace character, of newlines, of digits, base64
    blocks) under the DeepSeek-V3-shaped vocabulary: one replay and eight planned chunks against the oracle.
    The long runs are where that family's boundary rules walk furthest."""
    from graphtok_b200 import GTok, synth
    path = synth.vocab_path("cfg5")
    _, doc = synth.config_doc(4)
    want = oracle_lib.Oracle(path).encode_normalized(doc)
    g = GTok(path, max_bytes=len(doc) + 4096)
    try:
        assert np.array_equal(g.encode(doc), want)
        cuts = g.plan_chunks(doc, 8)
        parts = [g.encode(doc[int(cuts[k]):int(cuts[k + 1])]) for k in range(8)]
        assert np.array_equal(np.concatenate(parts), want)
    finally:
        g.close()


def test_gemma_vocabulary_on_large_documents(built):
    """The Gemma-3-shaped vocabulary on 4 MB of the multilingual text (a third of its characters are not in the
    3,000-token vocabulary and come out as byte tokens) and on 2 MB of the adversarial document (its long runs are long
    pre-tokens here): one replay and four planned chunks against the oracle, which merges each whole text without cutting it,
    and the ids decoded back."""
    from graphtok_b200 import GTok, synth
    path = tiny_vocab("gemma")
    o = oracle_lib.Oracle(path)
    for doc in (synth.text(1, 7, 4 << 20), synth.config_doc(4)[1][:2 << 20].decode("utf-8", "ignore").encode()):
        want = o.encode_normalized(doc)
        g = GTok(path, max_bytes=len(doc) + 4096)
        try:
            ids = g.encode(doc)
            assert np.array_equal(ids, want)
            cuts = g.plan_chunks(doc, 4)
            assert np.array_equal(np.concatenate([g.encode(doc[int(cuts[k]):int(cuts[k + 1])]) for k in range(4) if cuts[k + 1] > cuts[k]]), want)
            assert g.decode(ids) == decoded("gemma", doc)
        finally:
            g.close()


def test_configuration_2_batch_full_size(built):
    """All 8,192 documents of the batch configuration in one call: ids and per-document offsets
    against the oracle run document by document."""
    from graphtok_b200 import GTok, synth
    path, blob, offs = synth.config_batch()
    assert offs.size == 8193
    o = oracle_lib.Oracle(path)
    want_ids, want_doc = o.encode_batch(blob, offs)
    ref = _reference_or_none(path)
    if ref is not None:
        k = 1000                                    # the reference build on the first thousand documents
        ref_ids = np.concatenate([ref.encode_normalized(blob[int(offs[i]):int(offs[i + 1])]) for i in range(k)])
        assert np.array_equal(ref_ids, want_ids[:int(want_doc[k])])
    g = GTok(path, max_bytes=len(blob) + 4096)
    try:
        ids, doc = g.encode_batch(blob, offs)
        assert np.array_equal(ids, want_ids) and np.array_equal(doc, want_doc)
    finally:
        g.close()


def decoded(family, b):
    """What ids decode to when they were made from the bytes b: b itself, but for the Gemma-3 shape, whose U+2581 and
    space are one character of the vocabulary that decodes to a space."""
    return b.replace("\u2581".encode(), b" ") if family == "gemma" else b


@pytest.mark.parametrize("family", FAMILIES)
def test_decode_on_the_device(gtoks, oracles, family):
    """gtok_x_decode: random ids against the spellings read from the tokenizer.json, the golden
    texts back from their ids, encode -> decode round trips, sizes changing between calls."""
    g, o = gtoks[family], oracles[family]
    table = oracle_lib.token_spellings(tiny_vocab(family))
    known = np.array(sorted(table), dtype=np.uint32)
    rng = np.random.default_rng(6)
    for n in (1, 8, 9, 2047, 2048, 2049, 300000, 5, 70001):
        ids = rng.choice(known, size=n)
        assert g.decode(ids) == b"".join(table[int(t)] for t in ids), n
    data = json.load(open(os.path.join(GOLDEN, "golden_%s.json" % family)))
    for row in data["cases"]:
        assert g.decode(row["ids"]) == decoded(family, norm(o, row["text"].encode("utf-8"))), repr(row["text"][:40])
    for t in cases.fuzz_strings(78, SPECIAL[family], per_pool=40):
        b = norm(o, t.encode())
        if b:
            assert g.decode(g.encode(b)) == decoded(family, b), repr(t[:40])
    assert g.decode(np.zeros(0, dtype=np.uint32)) == b""
    longest = max(table, key=lambda t: len(table[t]))
    assert g.decode(np.full(50000, longest, dtype=np.uint32)) == table[longest] * 50000
    # thousands of tiles: more than are resident at once, a long look-back chain
    block = rng.choice(known, size=3001)
    assert g.decode(np.tile(block, 3000)) == b"".join(table[int(t)] for t in block) * 3000


def test_decode_return_codes_and_page_locked_output(gtoks):
    import torch
    g = gtoks["llama3"]
    table = oracle_lib.token_spellings(tiny_vocab("llama3"))
    ids = np.array(sorted(table)[:4000] * 10, dtype=np.uint32)
    want = b"".join(table[int(t)] for t in ids)
    need = ctypes.c_uint64(0)
    small = np.zeros(len(want) - 1, dtype=np.uint8)
    r = g.lib.gtok_x_decode(g.handle, ids.ctypes.data, ids.size, small.ctypes.data, small.size, ctypes.byref(need), None)
    assert r == -2 and need.value == len(want)
    r = g.lib.gtok_x_decode(g.handle, ids.ctypes.data, ids.size, None, 0, ctypes.byref(need), None)      # size query
    assert r == -2 and need.value == len(want)
    exact = np.zeros(len(want), dtype=np.uint8)
    r = g.lib.gtok_x_decode(g.handle, ids.ctypes.data, ids.size, exact.ctypes.data, exact.size, ctypes.byref(need), None)
    assert r == len(want) and exact.tobytes() == want
    pinned = torch.zeros(len(want) + 64, dtype=torch.uint8).pin_memory()
    arr = pinned.numpy()
    r = g.lib.gtok_x_decode(g.handle, ids.ctypes.data, ids.size, arr.ctypes.data, arr.size, None, None)
    assert r == len(want) and arr[:r].tobytes() == want and not arr[r:].any()
    bad = np.array([1, 2, 0x7FFFFFFF, 3], dtype=np.uint32)
    r = g.lib.gtok_x_decode(g.handle, bad.ctypes.data, bad.size, arr.ctypes.data, arr.size, None, None)
    assert r == -1 and b"outside the vocabulary" in g.lib.gtok_x_last_error()
    assert g.decode(ids[:100]) == b"".join(table[int(t)] for t in ids[:100])       # the handle still works


def test_decode_round_trip_full_size_configuration_1(built):
    """encode -> decode gives the document back, at the benchmark's size."""
    from graphtok_b200 import GTok, synth
    path, doc = synth.config_doc(1)
    g = GTok(path, max_bytes=len(doc) + 4096)
    try:
        ids = g.encode(doc)
        out, ms = g.decode(ids, want_ms=True)
        assert out == doc and 0 < ms < 50
    finally:
        g.close()


def test_python_module_surface(built, oracles):
    """The reference's Python classes over this library: same calls, same return types."""
    import gpu_bpe_tokenizer                                    # the reference's module name
    tok = gpu_bpe_tokenizer.Tokenizer(tiny_vocab("llama3"), max_input_chars=4096)
    handle_before = tok._g.handle
    o = oracles["llama3"]
    text = "Hello, world! It's 2026 <|reserved_special_token_3|> done"
    ids = tok.encode(text)
    assert isinstance(ids, list) and ids == o.encode(text.encode()).tolist() == tok(text)
    arr = tok.encode_numpy(text.encode())
    assert arr.dtype == np.uint32 and arr.tolist() == ids
    toks, offs = tok.encode_batch([text, "", "second doc"])
    assert toks.dtype == np.uint32 and offs.dtype == np.uint32 and offs.tolist()[0] == 0 and len(offs) == 4
    assert toks[offs[0]:offs[1]].tolist() == ids and offs[1] == offs[2]
    e_t, e_o = tok.encode_batch([])
    assert e_t.size == 0 and e_o.tolist() == [0]
    assert tok.decode(ids) == text and tok.decode_bytes(np.array(ids)) == text.encode()
    long_text = "grow " * 5000                                  # beyond max_input_chars: capacity grows
    assert tok.encode_numpy(long_text).tolist() == o.encode(long_text.encode()).tolist()
    assert tok._g.handle == handle_before                       # grown in place: same handle, same tables
    assert tok.active_capacity >= len(long_text) and tok.regex_kind == "Llama3" and tok.cpu_backend == "off" and tok.last_route == "gpu"
    assert tok.vocab_size > 256 and tok.host_max_bytes == 0
    dev = tok.encode_to_device(text)
    assert dev.is_cuda and dev.cpu().numpy().astype(np.uint32).tolist() == ids
    bt, bo = tok.encode_batch_to_device([text, "", "second doc"])
    assert bt.is_cuda and bo.is_cuda and bt.cpu().numpy().astype(np.uint32).tolist() == toks.tolist() and bo.cpu().tolist() == offs.tolist()
    tok.bench_stage(text)
    n, ms = tok.bench_run()
    assert n == len(ids) and ms >= 0
    with pytest.raises(ValueError):
        gpu_bpe_tokenizer.Dispatcher(tiny_vocab("gpt2"), policy="sometimes")
    d = gpu_bpe_tokenizer.Dispatcher(tiny_vocab("llama3"), cpu_workers=0, policy="gpu")
    assert d.encode_numpy(text).tolist() == ids and d.stats()["gpu_requests"] == 1 and d.stats()["gpu_batches"] == 1 and d.cpu_backend == "off"
    d.close()
