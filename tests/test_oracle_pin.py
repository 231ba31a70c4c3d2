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
    if family == "deepseek":
        pytest.skip("the reference has no host encoder for DeepSeek-V3 (src/host_encode.cc:951-953); Hugging Face is its pin")
    if family == "gemma":
        pytest.skip("the reference build used here is made without the Gemma-3 vocabulary (GBPE_HAVE_VOCAB_GEMMA3=0; its loader does "
                    "recognise the committed file as that shape); Hugging Face is the pin")
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
    ref_dir = oracle_lib.reference_dir()
    fx = os.path.join(ref_dir or "", "third_party", "rs-gigatoken", "tests", "fixtures", "gpt2_tokenizer.json")
    if not ref_dir or not os.path.exists(fx):
        pytest.skip("the reference tree (and its GPT-2 fixture) is not on this machine")
    o, ref = oracle_lib.Oracle(fx), oracle_lib.Reference(fx)
    for t in cases.fuzz_strings(3, "<|endoftext|>", per_pool=150) + ["Hello, world! It's 2026"]:
        assert np.array_equal(o.encode_normalized(t.encode()), ref.encode_normalized(t.encode())), repr(t[:60])
    assert o.encode_normalized(b"Hello, world! It's 2026").tolist() == [15496, 11, 995, 0, 632, 338, 1160, 2075]


@pytest.mark.parametrize("family", FAMILIES)
def test_oracle_boundaries_match_sequential_regex(oracles, built, family):
    """Pre-token starts from the oracle == starts from the cursor-based reading of the regex."""
    from graphtok_b200 import build
    if family == "gemma":
        pytest.skip("the Gemma-3 shape has no regular expression: its model merges the whole text, and where the kernels cut it is "
                    "checked by the ids (the oracle merges without cuts)")
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


def test_class_table_equals_the_references_table(built):
    """The two-bit class of every codepoint from this library's table (csrc/unicode_class_table.h, own
    two-stage layout) against the reference's generated table (generated/gbpe_class_table.h,
    gbpe_classify), over 0 .. 0x1FFFFF: every pre-tokenization predicate rests on it."""
    ref_dir = oracle_lib.reference_dir()
    if not ref_dir or not os.path.exists(os.path.join(ref_dir, "generated", "gbpe_class_table.h")):
        pytest.skip("the reference tree is not on this machine")
    src = r'''
#include "gbpe_class_table.h"
#include "unicode_class_table.h"
#include <cstdio>
int main() {
    long bad = 0;
    for (uint32_t cp = 0; cp < 0x200000; ++cp) {
        const uint32_t a = gbpe_classify(cp), b = gtok_uc_lookup(gtok_uc_stage1_init, gtok_uc_stage2_init, cp);
        if (a != b && bad++ < 10) std::printf("U+%X: reference %u, here %u\\n", cp, a, b);
    }
    std::printf("differences=%ld\\n", bad);
    return bad ? 1 : 0;
}
'''
    with tempfile.TemporaryDirectory() as d:
        cc, exe = os.path.join(d, "cmp.cc"), os.path.join(d, "cmp")
        with open(cc, "w") as f:
            f.write(src)
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ref_dir, "generated"), "-I", oracle_lib.CSRC, "-o", exe, cc], check=True)
        r = subprocess.run([exe], capture_output=True, text=True)
        assert r.returncode == 0 and "differences=0" in r.stdout, r.stdout


def test_wide_class_table_equals_the_references_bits(built):
    """The wide class of every codepoint (csrc/unicode_wide_table.h: letters and marks, numbers, whitespace,
    punctuation and symbols, other) against the reference's property bits (generated/gbpe_class_table.h:866-871,
    gbpe_class_bits), which must be mutually exclusive apart from nothing at all: the DeepSeek-V3 predicate
    rests on it."""
    ref_dir = oracle_lib.reference_dir()
    if not ref_dir or not os.path.exists(os.path.join(ref_dir, "generated", "gbpe_class_table.h")):
        pytest.skip("the reference tree is not on this machine")
    src = r'''
#include "gbpe_class_table.h"
#include "unicode_wide_table.h"
#include <cstdio>
int main() {
    long bad = 0;
    for (uint32_t cp = 0; cp < 0x200000; ++cp) {
        const uint32_t bits = cp <= 0x10FFFF ? gbpe_class_bits(cp) : 0u;
        int groups = 0;
        uint32_t want = 3;
        if (bits & (GBPE_WB_L | GBPE_WB_M)) { want = 0; ++groups; }
        if (bits & GBPE_WB_N) { want = 1; ++groups; }
        if (bits & GBPE_WB_WS) { want = 2; ++groups; }
        if (bits & (GBPE_WB_P | GBPE_WB_SY)) { want = 6; ++groups; }
        const uint32_t got = gtok_uw_lookup(gtok_uw_stage1_init, gtok_uw_stage2_init, cp);
        if ((groups > 1 || want != got) && bad++ < 10) std::printf("U+%X: reference bits %02x, here %u\\n", cp, bits, got);
    }
    std::printf("differences=%ld\\n", bad);
    return bad ? 1 : 0;
}
'''
    with tempfile.TemporaryDirectory() as d:
        cc, exe = os.path.join(d, "cmp.cc"), os.path.join(d, "cmp")
        with open(cc, "w") as f:
            f.write(src)
        subprocess.run(["g++", "-std=c++17", "-O1", "-DGBPE_HAVE_VOCAB_DEEPSEEK_V3=1", "-I", os.path.join(ref_dir, "generated"), "-I", oracle_lib.CSRC, "-o", exe, cc], check=True)
        r = subprocess.run([exe], capture_output=True, text=True)
        assert r.returncode == 0 and "differences=0" in r.stdout, r.stdout


def test_deepseek_oracle_against_tokenizers_live(oracles):
    """DeepSeek-V3 has no CPU encoder in the reference, so the oracle's reading of its three patterns is
    checked against Hugging Face `tokenizers` itself (the reference's own test oracle) on a seeded fuzz,
    beyond the committed golden vectors."""
    tokenizers = pytest.importorskip("tokenizers")
    hf = tokenizers.Tokenizer.from_file(tiny_vocab("deepseek"))
    o = oracles["deepseek"]
    texts = cases.fuzz_strings(21, SPECIAL["deepseek"], per_pool=400, lengths=(1, 2, 3, 5, 8, 13, 40, 120))
    for t in texts:
        assert o.encode(t.encode()).tolist() == hf.encode(t, add_special_tokens=False).ids, repr(t[:60])


def test_gemma_oracle_against_tokenizers_live(oracles):
    """The Gemma-3 shape has no host encoder in the reference build used here: the oracle's character-level merge loop against
    Hugging Face on fresh strings (spaces and U+2581, characters the vocabulary lacks, added tokens) and on slices of the synthetic text."""
    tokenizers = pytest.importorskip("tokenizers")
    import random
    from graphtok_b200 import synth
    hf = tokenizers.Tokenizer.from_file(tiny_vocab("gemma"))
    o = oracles["gemma"]
    rng = random.Random(31)
    pool = list("ab cd\n\t.,XY12\u2581") + ["\u00e9", "\u4e2d", "\u6587", "\U0001F600", "\u0301", "<bos>", "<eos>", "<pad", "  ", "   "]
    texts = ["".join(rng.choice(pool) for _ in range(rng.randint(1, 60))) for _ in range(1500)]
    doc = synth.text(1, 99, 200000).decode("utf-8", "ignore")
    texts += [doc[a:a + rng.randint(1, 600)] for a in (rng.randrange(len(doc) - 700) for _ in range(300))] + [doc[:40000]]
    for t in texts:
        assert o.encode_normalized(t.encode()).tolist() == hf.encode(t, add_special_tokens=False).ids, repr(t[:60])
