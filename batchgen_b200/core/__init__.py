"""Native (C++/CUDA) engine: weight slot ring + producer thread, node-shared host paged KV with prefix
coordinator, KV page movers, CPU decode attention.  Python front: ``core.native``."""
