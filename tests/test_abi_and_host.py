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


def test_loader_accepts_the_three_shapes_only(built):
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
    print("OK")
dist.destroy_process_group()
"""


def test_two_rank_document_sharding_with_gloo(built):
    """World size 2 on CPU: contiguous document ranges, all-gather of token counts, global offsets."""
    from graphtok_b200 import synth
    synth.config_batch(64, seed=9)      # generated once here, read by both ranks
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER % {"root": ROOT})
    try:
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                            "--master-port", "29731", f.name], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    finally:
        os.remove(f.name)
