"""`import gpu_bpe_tokenizer` -- the reference's module name (python/gpu_bpe_tokenizer/__init__.py:18-21)
for this repository's implementation of its classes over libgtok.so; see
graphtok_b200/gpu_bpe_tokenizer for the code."""
from graphtok_b200.gpu_bpe_tokenizer import Dispatcher, Tokenizer

__all__ = ["Tokenizer", "Dispatcher"]
