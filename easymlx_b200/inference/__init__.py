"""Serving-side helpers that sit next to the attention path."""
