"""Data-parallel machinery: process-group plumbing, flat buffers, the
communication engine (AllReducer) and the DistributedOptimizer wrapper."""
