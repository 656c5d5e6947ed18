"""Tokenizer toolchain: native pre-tokeniser / BPE trainer (C++), Python BPE trainer and encoder, dataset tokenisation."""
