"""Utilities: launch counting, tracing, graph visualisation."""
