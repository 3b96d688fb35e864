"""Benchmark/test harness around the hot path: seeded synthetic inputs and the network
forward passes assembled from the octree operators.  Not part of the drop-in operator API."""
