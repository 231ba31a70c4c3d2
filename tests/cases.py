"""Seeded input generators shared by the CPU and GPU parity tests."""
import random

import numpy as np

TILE = 4096          # tile of the words / assemble kernels
PTILE = 8000         # tile of the pre-tokenization kernel (its window of 8192 bytes less the halos)

POOLS = {
    "mixed": list("ab cd\r\n1.'sXY tlrevmTLREVM\t") + ["é", "日", "ſ", " ", "2", "'ll", "'RE", "\n\n", "  ", "!!"],
    "space": list("a \n\r.") + [" ", " ", "　", "\t"],
    "digit": list("0123456789 a.") + ["٣", "५"],
    "apos": list("'stdmlrve ") + ["ſ", "'"],
    # punctuation and symbols, marks, the CJK ranges and codepoints of no class: what the DeepSeek-V3 patterns tell apart
    "wide": list("ab Z!.-$_ \n\r\t") + ["é", "\u0301", "中", "文", "の", "カ", "・", "゛", "\x00", "\x01", "\u200b", "…", "«", "€", "1", "12", "٣",
                                       "\u00a0", "!a", " !", "a.b", "ａ"],
}


def fuzz_strings(seed, special, per_pool=300, lengths=(1, 2, 3, 5, 8, 13, 40, 120, 700)):
    rng = random.Random(seed)
    out = []
    for name, pool in POOLS.items():
        pool = list(pool)
        if special:
            pool += [special, "<", "|", "<|"]
        for _ in range(per_pool):
            n = rng.randint(1, rng.choice(lengths))
            out.append("".join(rng.choice(pool) for _ in range(n)))
    return out


def malformed_bytes(seed, count=300):
    rng = random.Random(seed)
    alphabet = [0x61, 0x20, 0x80, 0xBF, 0xC3, 0xE4, 0xF0, 0xA9, 0x0A, 0x27, 0x73, 0x31, 0xFF, 0xC5, 0x2E]
    out = [bytes(rng.choice(alphabet) for _ in range(rng.randint(1, 60))) for _ in range(count)]
    # stray continuation bytes for longer than the pre-tokenization window, before and after other text
    out += [b"a" + b"\x80" * 9000 + b"b c", b"\xbf" * 9000 + b"'s", b"a \xe4" + b"\x80\xbf" * 4500 + b" 12", b"x\n" + b"\x80" * 9000 + b"\n y",
            b"a" + b"\x80" * 17 + b"b" + b"\xa9" * 8200 + b"1234"]
    return out


def tile_crossers(special):
    """Inputs whose interesting structure sits on tile edges (4096-byte and 8000-byte tiles, 128/64-byte halos)."""
    out = []
    for pad in (TILE - 70, TILE - 3, TILE - 2, TILE - 1, TILE, TILE + 1, 2 * TILE - 1):
        base = ("ab " * (pad // 3 + 1))[:pad]
        for mid in (" " * 300, "\n" * 300, " \n" * 150, "\n " * 150, "." + "\n" * 200 + " x", "7" * 500, "7" * 9000, "x" * 20, "x" * 5000,
                    "don't", "'ll", " 's", "é" * 100, "日本語" * 50, ".\r\n\r\n  \r\n y", "a" + " " * 129 + "\n" + " " * 200 + "b", "\t" * 70 + "z",
                    "=" * 200 + "\n\n\n" + "w", "1 2 3 4 5 6 7 8 9 " * 30):
            out.append(base + mid + " tail end.")
            if special:
                out.append(base + special + mid + special + special + " t")
    # the same kinds of structure on the edges of the pre-tokenization kernel's own tiles
    for pad in (PTILE - 70, PTILE - 2, PTILE - 1, PTILE, PTILE + 1):
        base = ("ab " * (pad // 3 + 1))[:pad]
        for mid in (" " * 300, " \n" * 150, "." + "\n" * 200 + " x", "7" * 500, "x" * 20, "don't", "'ll", "é" * 100, "日本語" * 50, ".\r\n\r\n  \r\n y",
                    "1 2 3 4 5 6 7 8 9 " * 30):
            out.append(base + mid + " tail end.")
            if special:
                out.append(base + special + mid + special + special + " t")
    if special:
        # more literals in one tile than are looked up in parallel, and literals cut by the end of the text
        out.append("a" + special * 130 + " x " + special * 30 + special[:-1])
        out.append((special + ".") * 70)
    # run walks that leave the tile window (plain whitespace right after a very long newline stretch,
    # and a very long stretch of spaces right after a newline)
    for head in ("a", ".", "1", ""):
        out.append("lead " + head + "\n" * 9000 + "  x")
        out.append("lead " + head + "\r\n" * 4500 + " \tx")
        out.append("lead " + head + "\n" * 9000 + " " * 9000 + "x")
    out.append("k\n" + " " * 9000 + "x")
    out.append("k\n" + " " * 9000 + "\n x")
    out.append("k\n" + " " * 9000)
    out.append("k\n" + " " * 5000 + "\t" + " " * 5000 + "\n\nq")
    out.append("k\n" + "\t" * 9000 + "\nq")
    out.append("k\n" + "\t" * 9000 + "q")
    out.append("k\n" + "\u00a0" * 5000 + "q")
    out.append("k\n" + "\u3000\t " * 3000 + "\nq")
    out.append("k!" + "\n" * 9000 + " q")
    out.append("\n" * 9000 + " q")
    # ASCII letters behind a punctuation mark, or not, for longer than the window, then another kind of letter
    # (the first alternative of the DeepSeek-V3 main pattern stops there)
    for head in ("!", " !", "!!", "", "x.", "1", "中", "\n"):
        out.append("w " + head + "a" * 9000 + "é b")
        out.append(head + "Zq" * 4500 + "\u0301 b")
    # long pre-tokens made of a few byte runs (run-length merge path) and of many (general path)
    out.append("w " + "a" * 3000 + "b" * 3000 + "a" * 10 + " t")
    out.append("w " + "=" * 700 + "-" * 65 + "=" * 2 + "~" * 9000 + " t")
    out.append("w" + (" " * 70 + "\t" * 70) * 3 + "t")
    out.append("w " + "ab" * 40 + " " + "abc" * 2000 + " t")
    # long pre-tokens that are no handful of runs: merged in pieces of at most 64 bytes whose cuts are checked
    # (random text over small and large alphabets), or by the general path when a cut fails (periodic text)
    rng = random.Random(4242)
    for alphabet, length in (("abcdefghijklmnopqrstuvwxyz", 20000), ("ACGT", 9000), ("etaoinshr", 3000), ("ab", 700), ("theinandofto", 5000),
                             ("中文日本語的一是不了人我在有他这为之大来以个", 2500), ("éèêàùç", 900), ("!@#$%^&*()-=+", 4000)):
        out.append("p " + "".join(rng.choice(alphabet) for _ in range(length)) + " q")
    # many pre-tokens of 17 to 32 bytes that are no vocabulary tokens (what one block does not merge itself it hands back),
    # alone and among ones that may be
    b64 = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/"
    out.append(" ".join("".join(rng.choice(b64[:52]) for _ in range(rng.randint(17, 32))) for _ in range(900)))
    out.append(" ".join(("".join(rng.choice(b64[:52]) for _ in range(rng.randint(14, 34))) if rng.random() < 0.6 else
                         rng.choice(("international", "responsibilities", "internationalization", "characteristically", "telecommunications")))
                        for _ in range(1500)))
    out.append("p " + "the" * 600 + "in" * 500 + " q")
    out.append("p " + "thequickbrownfox" * 200 + " q")
    out.append("é" * 3000 + "日" * 2000 + "\U0001F600" * 500)
    out.append("z" * (3 * TILE + 17))
    out.append("9" * (2 * TILE + 5) + " " + "8" * 100)
    out.append((" " * (TILE + 100)) + "x")
    out.append(("\n" * (TILE + 100)) + "x")
    out.append("ab" * 1100 + " q")
    out.append("abcde" * 2500)
    return out


def length_ladder():
    out = []
    for n in (1, 2, 15, 16, 17, 18, 31, 32, 33, 47, 48, 49, 50, 63, 64, 65, 129, 257, 513, 1025, 1529, 1530, 1531, 2048, 2049, 4095, 4096, 4097, 9000):
        out += ["a" * n, "ab" * (n // 2 + 1), ("the" * (n // 3 + 1))[:n], "x " + "q" * n + " y"]
    return out


def make_batch(seed, docs_text):
    """Concatenation + uint32 offsets, with a few empty documents mixed in."""
    rng = random.Random(seed)
    blobs, offs = [], [0]
    for t in docs_text:
        b = t if isinstance(t, bytes) else t.encode("utf-8")
        if rng.random() < 0.15:
            offs.append(offs[-1])      # an empty document first
        blobs.append(b)
        offs.append(offs[-1] + len(b))
    return b"".join(blobs), np.array(offs, dtype=np.uint32)


SEAM_DOCS = [
    "123", "456", "12", "3456789", " ", "  ", "a ", " b", "\n", "\r", "\n\n", "x\r", "\ny", "don", "'t", "'", "s", "it'", "ll go",
    ".", "\n.", ".\n", "\n", "a.", "\n\nb", "é", "e", "́", "日本", "語", "x  ", "  y", "\t", "\tz", "", "", "end",
]
