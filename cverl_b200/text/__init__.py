"""Tokenizers over the native host library: byte-level and Hugging Face byte-level BPE."""
from .tokenizer import ByteTokenizer, EncodeOptions, HfBpeTokenizer, Tokenizer  # noqa: F401
