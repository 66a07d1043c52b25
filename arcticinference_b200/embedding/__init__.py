"""Embedding service: encoder engine, gRPC replica, replica manager and client."""

from .engine import AsyncEmbeddingEngine, EmbeddingEngine  # noqa: F401
