"""Replica-pool serving: REST API, request scheduler, workers, metrics, weight sync."""
