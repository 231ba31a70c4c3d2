"""The three CPU encoders on the benchmark configurations at their stated sizes: this repository's
oracle (oracle/gtok_oracle.cc), the reference's own host encoder compiled from its sources
(oracle/_ref, when a checkout of the reference is present) and Hugging Face `tokenizers`
(the reference's own test oracle) must give the same ids.  The GPU tests then compare the kernels
with the oracle on the same documents."""
import numpy as np
import pytest

import oracle_lib

pytestmark = pytest.mark.slow


def _hf(path):
    tokenizers = pytest.importorskip("tokenizers")
    return tokenizers.Tokenizer.from_file(path)


def _hf_ids(hf, data):
    return np.array(hf.encode(data.decode("utf-8"), add_special_tokens=False).ids, dtype=np.uint32)


def _ref(path):
    return oracle_lib.Reference(path) if oracle_lib.build_ref() else None


@pytest.mark.parametrize("config", (0, 1, 3, 5))
def test_single_document_configurations(built, config):
    """(5 is the DeepSeek-V3-shaped vocabulary, for which the reference has no host encoder: two-way.)"""
    from graphtok_b200 import synth
    path, doc = synth.config_doc(config)
    o = oracle_lib.Oracle(path)
    want = o.encode(doc)                                   # normalises first where the vocabulary declares NFC
    assert np.array_equal(_hf_ids(_hf(path), doc), want)   # Hugging Face normalises by itself
    ref = _ref(path) if config != 5 else None
    if ref is not None:
        assert np.array_equal(ref.encode_normalized(oracle_lib.nfc(doc) if o.needs_nfc else doc), want)


def test_batch_configuration(built):
    from graphtok_b200 import synth
    path, blob, offs = synth.config_batch()
    o = oracle_lib.Oracle(path)
    want_ids, want_doc = o.encode_batch(blob, offs)
    docs = [blob[int(offs[i]):int(offs[i + 1])].decode("utf-8") for i in range(offs.size - 1)]
    got = _hf(path).encode_batch(docs, add_special_tokens=False)
    assert np.array_equal(np.concatenate([np.array(e.ids, dtype=np.uint32) for e in got]), want_ids)
    assert np.array_equal(np.cumsum([0] + [len(e.ids) for e in got]), want_doc)
    ref = _ref(path)
    if ref is not None:
        ref_ids = np.concatenate([ref.encode_normalized(blob[int(offs[i]):int(offs[i + 1])]) for i in range(offs.size - 1)])
        assert np.array_equal(ref_ids, want_ids)


def test_adversarial_configuration(built):
    """32 MB: oracle against the reference's encoder on the whole document; Hugging Face (a minute
    on the whole) on the first 8 MB, which holds every kind of block the document is made of."""
    from graphtok_b200 import synth
    path, doc = synth.config_doc(4)
    o = oracle_lib.Oracle(path)
    ref = _ref(path)
    if ref is not None:
        assert np.array_equal(ref.encode_normalized(doc), o.encode_normalized(doc))
    pre = doc[:8 << 20].decode("utf-8", "ignore").encode()
    assert np.array_equal(_hf_ids(_hf(path), pre), o.encode_normalized(pre))
