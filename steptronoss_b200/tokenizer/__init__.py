"""Tokenizer front-end with a stable contract across Hugging Face releases."""
from .hf_compat_tokenizer import BaseTokenizer, HFCompatTokenizer, load_hf_tokenizer  # noqa: F401
