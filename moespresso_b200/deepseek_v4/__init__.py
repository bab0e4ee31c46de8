"""DeepSeek-V4-shaped attention operators (indexer score, top-k, indexed sparse attention)."""
