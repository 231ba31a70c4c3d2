"""The command-line tool (graphtok_b200/cli/gpu_bpe_tokenize) writes the reference tool's output files:
flat uint32 ids for one document, [n_docs][doc_off x (n_docs+1)][ids] for a batch
(src/main.cc:531-549 of the reference), [n_runs][offsets x (n_runs+1)][ids] for a benchmark list
(src/main.cc:397-419), and the bytes of decoded ids.  Contents are checked against the CPU oracle."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import oracle_lib
from conftest import tiny_vocab

pytestmark = pytest.mark.gpu


def _run(args):
    from graphtok_b200 import build
    r = subprocess.run([build.build_cli()] + args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1500:]
    return r.stdout


def test_cli_output_files(built):
    vocab = tiny_vocab("llama3")
    o = oracle_lib.Oracle(vocab)
    docs = [b"Hello, world! It's 2026 <|reserved_special_token_3|> done", b"", "café 日本語 12345 ".encode() * 40, b"third document\n\n  indented"]
    with tempfile.TemporaryDirectory() as d:
        paths = []
        for i, t in enumerate(docs):
            p = os.path.join(d, "doc%d.txt" % i)
            open(p, "wb").write(t)
            paths.append(p)
        want = [o.encode(t) for t in docs]
        out = os.path.join(d, "out.bin")
        # one document: flat ids; CSV header and one line per run
        csv = _run(["--vocab", vocab, "--input", paths[2], "--output", out, "--runs", "2", "--warmup", "1", "--csv"])
        assert np.array_equal(np.fromfile(out, dtype=np.uint32), want[2])
        lines = csv.strip().splitlines()
        assert lines[0] == "run,n_tokens_out,n_pretokens,pretok_ms,kernel_ms,e2e_ms,full_e2e_ms" and len(lines) == 3
        assert int(lines[1].split(",")[1]) == want[2].size
        # batch
        csv = _run(["--vocab", vocab, "--inputs", ",".join(paths), "--output", out, "--csv"])
        raw = np.fromfile(out, dtype=np.uint32)
        n_docs = int(raw[0])
        assert n_docs == len(docs)
        doc_off = raw[1:n_docs + 2]
        assert doc_off.tolist() == np.concatenate([[0], np.cumsum([w.size for w in want])]).tolist()
        assert np.array_equal(raw[n_docs + 2:], np.concatenate(want))
        assert csv.splitlines()[0] == "run,n_docs,n_tokens_out,kernel_ms,e2e_ms"
        # benchmark list: run i encodes input i mod n
        listing = os.path.join(d, "list.txt")
        open(listing, "w").write("\n".join([paths[0], paths[2], paths[3]]) + "\n")
        _run(["--vocab", vocab, "--benchmark-input-list", listing, "--output", out, "--runs", "5"])
        raw = np.fromfile(out, dtype=np.uint32)
        assert int(raw[0]) == 5
        offs = raw[1:7]
        order = [want[0], want[2], want[3], want[0], want[2]]
        assert offs.tolist() == np.concatenate([[0], np.cumsum([w.size for w in order])]).tolist()
        assert np.array_equal(raw[7:], np.concatenate(order))
        # decode: ids back to the document's bytes
        ids_file = os.path.join(d, "ids.bin")
        want[2].astype(np.uint32).tofile(ids_file)
        _run(["--vocab", vocab, "--decode", "--input", ids_file, "--output", out])
        assert open(out, "rb").read() == docs[2]
