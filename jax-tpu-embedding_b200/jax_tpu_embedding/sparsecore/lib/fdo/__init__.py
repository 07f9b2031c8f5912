"""Feedback-directed optimisation clients: they persist the statistics that input preprocessing
reports so that later runs can size limits and buffers from observed data."""
