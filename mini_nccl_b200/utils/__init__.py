"""Utilities: host oracles and data generators, device timing, clock sampling."""
