"""Timing-based (spike-time coded) neurons and encoders."""
