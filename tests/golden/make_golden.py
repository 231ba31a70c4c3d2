#!/usr/bin/env python3
"""Regenerates the golden vectors in this directory.

Vocabularies: tiny_{gpt2,llama3,qwen25,deepseek}.json, written by the in-tree generator
(graphtok_b200.synth.vocab_path("tiny_*"): seeded corpus + greedy BPE trainer) and
committed here because the expected ids are only meaningful for these exact files.
tiny_gemma.json (the Gemma-3 shape: characters merged by a SentencePiece-style BPE, spaces
written as U+2581, byte fallback) is made by make_tiny_gemma() below with the `tokenizers`
trainer on the in-tree synthetic text; `--vocab` rewrites it, else the committed file is used.

Expected ids: Hugging Face `tokenizers` (the reference's own test oracle,
tests/test_encode_batch.py:69-84 there) on every case string:
    Tokenizer.from_file(vocab).encode(text, add_special_tokens=False).ids
For the Qwen2.5-shaped vocabulary that call includes the file's NFC normaliser.

The case list follows the shapes of the reference's tests: document-seam strings
(tests/seam_corpus.py), pre-token lengths around the bucket cut-overs
(tests/test_exactness_targeted.py:39,83-88), equal-rank runs (:104-124),
added-token edge strings (tests/test_host_fast_path.py:107-128), a small-alphabet
fuzz (:132-141) and the named NFC cases (tests/test_nfc_normalization.py).

Run:  python tests/golden/make_golden.py        (needs `tokenizers`; offline)
"""
import json
import os
import random

from tokenizers import Tokenizer

HERE = os.path.dirname(os.path.abspath(__file__))


def cases(family, special):
    c = [
        "", " ", "  ", "\n", "\r\n", "a", "Hello, world! It's 2026", "don't DON'T can't he'll we're I've I'm she'd 'tis",
        "x'sy 'll 'LL ''s .'s  's \t's a'", "'s", "'", "''", "a'\nb", "1'st 2'nd",
        "tabs\tand\t\tmore \t mixed", "trailing spaces   ", "   leading", "line1\nline2\n\nline4\r\n\r\nline6",
        "code:\n    if (x == 1) {\n        return y[i];\n    }\n", "a.\n\nb", "a.\r\n \r\n b", "x !\n\n  y", "x;\n\t\ty",
        "1 12 123 1234 12345 123456 1234567 12345678901234567890", "3.14159 1,000,000 0x1F 1e-9", "٣٤٥٦٧ ५६७८ ①②③④",
        "ünïcödé Ωmega привет мир Ελληνικά", "日本語のテキスト 中文文本 한국어", "emoji 🙂🙃 👍🏽 done", "a\u00a0b\u2003c\u3000d\u2028e",
        "ſ 'ſ x'ſy İstanbul ǅ", "(word) -word --word \"quoted\" [x]{y}<z>", "a+b=c; d->e; f::g; #h @i $j %k ^l &m *n",
        "aaaaaaaaaaaaaaa", "a" * 16, "a" * 17, "a" * 31, "a" * 32, "a" * 33, "a" * 63, "a" * 64, "a" * 65, "a" * 129, "a" * 257,
        "a" * 513, "a" * 1025, "ab" * 600, "abc" * 700, " " * 100, "\n" * 100, " \n" * 60, "x" + " " * 70 + "y", "x" + "\n" * 70 + "y",
        "." * 90, ".\n" * 50, "=" * 300, "9" * 400, "z" * 2100, "mn" * 2600,
        "the quick brown fox jumps over the lazy dog " * 40,
        "https://example.com/a/b/c?d=e&f=g#h user@example.org C:\\path\\file.txt",
        "supercalifragilisticexpialidocious antidisestablishmentarianism pneumonoultramicroscopicsilicovolcanoconiosis",
        "中" * 40, "日本" * 300, "é" * 50, "e\u0301" * 50, "🙂" * 30,
    ]
    if special:
        s = special
        c += [s, s + s, "a" + s + "b", " " + s + " ", s + "'s", "x" + s + "\n\n" + s + " y", "<" + s, s[:-1], s[:-1] + " " + s,
              "<|" + s, "12" + s + "345", "a " + s + "  " + s + " b", s + "é", "\n" + s + "\n"]
    rng = random.Random(20260101)
    pools = [list("ab cd\r\n1.'sXY"), list("'stdmlrve LRVE\t"), list("0123456789 ,."), list(" \n\r\t.x")]
    for pool in pools:
        for _ in range(120):
            c.append("".join(rng.choice(pool) for _ in range(rng.randint(1, 48))))
    if family == "deepseek":
        # the first alternative (a punctuation mark taking ASCII letters along) and what stops it; the three CJK
        # ranges; marks; codepoints of no class; whitespace against the ends of pieces
        c += ["!abc", "a.b.c", " !abc", "!!ab", "a!b!c", "!ab\u00e9", "!ab\u00e9cd", ".ab1cd", "x$yz", "\t!a", "\n!a", "!a\n", "_a_b", "a\u0301!b",
              "\u4e2d\u6587abc\u4e2d\u6587", "\u4e2d\u6587 abc", "abc \u4e2d", "\u3042\u30a2\u4e00", "\u30fb\u30fc\u309b\u3099", "\u4e001\u4e00", "\u9fa5\u9fa6", "\u303f\u3040\u30ff\u3100",
              "\u0301", "\u0301a", "a\u0301\u0302b", " \u0301", "\u0301 \u0301",
              "\x00", "\x00\x01", "\x00a", "\x00\x01a", "a\x00b", "\x00 ", " \x00", "\u200b\u200bx", "!\x00", "\x00!", "\x00\n",
              "a  1", "a 1", "  1", "1  a", "1 a", "12  ", "  \u4e2d", " \u4e2d", "\u4e2d  a", "a\n 1", "a \n1", "!\n\n 1", "!\n \n x", "a\n \n x", " \n \n", "\n \n  ",
              "1234567", "12a345", "\u0663\u0664\u0665\u0666", "1\u00b22", "3.14159", "1,000,000", "\u2460\u2461\u2462\u2463",
              " \u00a0a", "\u00a0 a", "\u3000a", "a\u2028b", "\u0085a", "\x1ca", "\x0bx \x0c y"]
        rng2 = random.Random(20260102)
        pool = list("ab Z!.-$_ \n\r\t") + ["\u00e9", "\u0301", "\u4e2d", "\u6587", "\u306e", "\u30ab", "\u30fb", "\u309b", "\x00", "\x01", "\u200b", "\u2026", "\u00ab", "\u20ac", "1", "12", "\u0663", "\u00a0"]
        for _ in range(400):
            c.append("".join(rng2.choice(pool) for _ in range(rng2.randint(1, 40))))
    if family == "gemma":
        # spaces against U+2581 itself, characters the vocabulary lacks (byte fallback), runs of spaces
        c += ["\u2581", " \u2581 ", "a\u2581b c", "\u2581\u2581x", "x \u2581", "\u4e2d\u6587 \u6587\u4e2d", "\U0001F600 \U0001F600", "a\u0301 b\u0301",
              "\x00 \x01", "\x7f", "word<eos>word", "<bos> x", "x <bos>", "<bo s>", " <pad>"]
        rng3 = random.Random(20260103)
        pool = list("ab cd\n\t.,XY12\u2581") + ["\u00e9", "\u4e2d", "\u6587", "\U0001F600", "\u0301", "<bos>", "<eos>", "  ", "   "]
        for _ in range(500):
            c.append("".join(rng3.choice(pool) for _ in range(rng3.randint(1, 40))))
    if family == "qwen25":
        c += ["e\u0301", "a\u0308o\u0308u\u0308", "\u0041\u030a", "\u212b", "\u1e9b\u0323", "q\u0307\u0323", "\uac00", "\u1100\u1161\u11a8",
              "\u0958", "\u0b47\u0b56", "x\u0301\u0301\u0301", "\u0301a", "caf\u0065\u0301 na\u0069\u0308ve", "\ufb01 \u00bd \u2126",
              "a\u0323\u0302", "\u0f73", "\u1f71", "\u2000\u2001", "\u0344", "D\u0307\u0323", "\u1ebf", "e\u0302\u0301", "\u09cb", "\u09c7\u09be"]
    seen, out = set(), []
    for s in c:
        if s not in seen:
            seen.add(s)
            out.append(s)
    return out


def make_tiny_gemma(path):
    """A small vocabulary of the Gemma-3 shape: trained on pieces that do not cross a space (as SentencePiece does),
    then given the file's real sections (Replace normaliser, the Split on " ", byte-fallback tokens, the decoder)."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from tokenizers import Regex, models, normalizers, pre_tokenizers, trainers
    from graphtok_b200 import synth
    text = synth.text(1, 4242, 600000).decode("utf-8", "ignore")
    tok = Tokenizer(models.BPE(unk_token="<unk>", byte_fallback=True, fuse_unk=True))
    tok.normalizer = normalizers.Replace(" ", "\u2581")
    tok.pre_tokenizer = pre_tokenizers.Split(Regex("\u2581"), behavior="merged_with_next")
    specials = ["<pad>", "<eos>", "<bos>", "<unk>"]
    tok.train_from_iterator([l for l in text.split("\n") if l],
                            trainers.BpeTrainer(vocab_size=3000, special_tokens=specials, show_progress=False, limit_alphabet=400))
    j = json.loads(tok.to_str())
    vocab = j["model"]["vocab"]
    nid = max(vocab.values()) + 1
    for b in range(256):
        vocab["<0x%02X>" % b] = nid + b
    j["normalizer"] = {"type": "Replace", "pattern": {"String": " "}, "content": "\u2581"}
    j["pre_tokenizer"] = {"type": "Split", "pattern": {"String": " "}, "behavior": "MergedWithPrevious", "invert": False}
    j["decoder"] = {"type": "Sequence", "decoders": [{"type": "Replace", "pattern": {"String": "\u2581"}, "content": " "},
                                                     {"type": "ByteFallback"}, {"type": "Fuse"}]}
    j["post_processor"] = None
    j["added_tokens"] = [{"id": vocab[s], "content": s, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False,
                          "special": True} for s in specials]
    with open(path, "w") as f:
        json.dump(j, f, ensure_ascii=False)


def main():
    import sys
    if "--vocab" in sys.argv:
        make_tiny_gemma(os.path.join(HERE, "tiny_gemma.json"))
    for family, special in (("gpt2", None), ("llama3", "<|reserved_special_token_3|>"), ("qwen25", "<|qwen_special_1|>"),
                            ("deepseek", "<\uff5cspecial\u25811\uff5c>"), ("gemma", "<bos>")):
        vocab = os.path.join(HERE, "tiny_%s.json" % family)
        tok = Tokenizer.from_file(vocab)
        rows = []
        for s in cases(family, special):
            rows.append({"text": s, "ids": tok.encode(s, add_special_tokens=False).ids})
        with open(os.path.join(HERE, "golden_%s.json" % family), "w") as f:
            json.dump({"vocab": "tiny_%s.json" % family, "source": "tokenizers " + __import__("tokenizers").__version__, "cases": rows}, f, ensure_ascii=True)
        print(family, len(rows), "cases")


if __name__ == "__main__":
    main()
