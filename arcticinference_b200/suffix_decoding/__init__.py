"""Suffix decoding: model-free speculation from suffix trees over past and current
sequences (global tree of finished responses + one tree per running request)."""

from .cache import SuffixDecodingCache, SuffixDecodingDraft

__all__ = ["SuffixDecodingCache", "SuffixDecodingDraft"]
