"""Operators: torch restatements of the codecs and algorithms (codecs), the error-bounded codec and
its container (sz), stand-alone codec kernels (standalone)."""
