"""Worker runtime: sequences, paged KV, schedulers, engine, CUDA graphs, offline batch API."""
