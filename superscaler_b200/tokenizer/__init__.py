"""Tokenizers: GPT-2 byte-level BPE, BERT WordPiece, and the vocabulary-size padding rule the models use."""
from .tokenizer import BertWordPieceTokenizer, GPT2BPETokenizer, build_tokenizer, padded_vocab_size  # noqa: F401
