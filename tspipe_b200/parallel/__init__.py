"""Data-parallel pieces layered on the pipeline: key all-gather, replica helpers."""
