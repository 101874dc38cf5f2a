"""Dataset converters (downloaded dataset files -> prompt records)."""
