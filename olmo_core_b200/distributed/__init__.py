"""Distributed runtime: process-group bootstrap, rank helpers, meshes and parallelism configs."""
