"""Parallelism runtime: process-group topology, ZeRO-3 engine, TP / PP / CP / EP."""
