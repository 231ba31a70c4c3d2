"""Pins the CPU oracle: against golden vectors from Hugging Face `tokenizers`, against the
reference's own host encoder when it was built from its sources, and against the sequential
regex reading used by the vocabulary trainer."""
import json
import os
import subprocess
import tempfile

import numpy as np
import pytest

import oracle_lib
from conftest import FAMILIES, GOLDEN, SPECIAL, tiny_vocab
import cases


@pytest.mark.parametrize("family", FAMILIES)
def test_oracle_matches_golden(oracles, family):
    data = json.load(open(os.path.join(GOLDEN, "golden_%s.json" % family)))
    o = oracles[family]
    bad = []
    for row in data["cases"]:
        got = o.encode(row["text"].encode("utf-8")).tolist()
        if got != row["ids"]:
            bad.append(row["text"][:40])
    assert not bad, "oracle differs from Hugging Face tokenizers on %d cases, e.g. %r" % (len(bad), bad[:3])


@pytest.mark.parametrize("family", FAMILIES)
def test_oracle_matches_reference_build(oracles, family):
    try:
        ref = oracle_lib.Reference(tiny_vocab(family))
    except FileNotFoundError:
        pytest.skip("reference host encoder not built (its sources are not on this machine)")
    o = oracles[family]
    texts = cases.fuzz_strings(5, SPECIAL[family], per_pool=250) + cases.length_ladder() + cases.tile_crossers(SPECIAL[family])[:40]
    for t in texts:
        b = oracle_lib.nfc(t.encode()) if o.needs_nfc else t.encode()
        assert np.array_equal(o.encode_normalized(b), ref.encode_normalized(b)), repr(t[:60])
    for b in cases.malformed_bytes(9, 300):
        assert np.array_equal(o.encode_normalized(b), ref.encode_normalized(b)), repr(b)


def test_oracle_matches_reference_on_real_gpt2_vocab(built):
    fx = "/root/reference/third_party/rs-gigatoken/tests/fixtures/gpt2_tokenizer.json"
    if not os.path.exists(fx):
        pytest.skip("the reference tree (and its GPT-2 fixture) is not on this machine")
    o, ref = oracle_lib.Oracle(fx), oracle_lib.Reference(fx)
    for t in cases.fuzz_strings(3, "<|endoftext|>", per_pool=150) + ["Hello, world! It's 2026"]:
        assert np.array_equal(o.encode_normalized(t.encode()), ref.encode_normalized(t.encode())), repr(t[:60])
    assert o.encode_normalized(b"Hello, world! It's 2026").tolist() == [15496, 11, 995, 0, 632, 338, 1160, 2075]


@pytest.mark.parametrize("family", FAMILIES)
def test_oracle_boundaries_match_sequential_regex(oracles, built, family):
    """Pre-token starts from the oracle == starts from the cursor-based reading of the regex."""
    from graphtok_b200 import build
    o = oracles[family]
    texts = [t for t in cases.fuzz_strings(11, None, per_pool=150) if t]
    with tempfile.TemporaryDirectory() as d:
        for i, t in enumerate(texts):
            b = oracle_lib.nfc(t.encode()) if o.needs_nfc else t.encode()
            open(os.path.join(d, "t.bin"), "wb").write(b)
            subprocess.run([build.build_datagen(), "split", family, os.path.join(d, "t.bin"), os.path.join(d, "s.bin")], check=True)
            want = np.fromfile(os.path.join(d, "s.bin"), dtype=np.uint32)
            _, got = o.encode_normalized(b, want_starts=True)
            assert np.array_equal(got, want), repr(t[:60])
            if i > 250:
                break
