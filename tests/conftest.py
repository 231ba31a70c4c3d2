import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

GOLDEN = os.path.join(ROOT, "tests", "golden")
FAMILIES = ("gpt2", "llama3", "qwen25", "deepseek", "gemma")
SPECIAL = {"gpt2": None, "llama3": "<|reserved_special_token_3|>", "qwen25": "<|qwen_special_1|>", "deepseek": "<\uff5cspecial\u25811\uff5c>", "gemma": "<bos>"}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")
    config.addinivalue_line("markers", "slow: CPU tests on the full-size configurations (a minute or two in all)")


def tiny_vocab(family):
    return os.path.join(GOLDEN, "tiny_%s.json" % family)


@pytest.fixture(scope="session")
def built():
    """Native pieces built once per session (libgtok, datagen, oracle, emulation, reference if present)."""
    import __graft_entry__
    __graft_entry__.build()
    return True


@pytest.fixture(scope="session")
def oracles(built):
    import oracle_lib
    return {f: oracle_lib.Oracle(tiny_vocab(f)) for f in FAMILIES}


@pytest.fixture(scope="session")
def emuls(built):
    import oracle_lib
    return {f: oracle_lib.Emul(tiny_vocab(f)) for f in FAMILIES}
