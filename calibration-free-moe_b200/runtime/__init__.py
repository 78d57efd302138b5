"""Callers of the reader inside a serving engine: decode/prefill row split, chunking, reports."""
