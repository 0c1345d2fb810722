"""Command-line tools: checkpoint conversion between HuggingFace files and the per-block layout."""
